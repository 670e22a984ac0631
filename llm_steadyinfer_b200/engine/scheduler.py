"""Continuous-batching scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees. Host logic only; it talks to the cache manager and hands
the step function a list of (request, next tokens, want logits).

State machine and policies follow the reference's ``Scheduler``
(src/source/scheduler/scheduler.cpp): WAITING -> RUNNING -> {PREEMPTED -> RUNNING}* -> FINISHED
(src/include/scheduler/sequence.h:12-18); first-come-first-served admission that reserves the
prompt's pages (scheduler.cpp:194-249); decode rows first, then prompt portions in admission
order under the budget (:378-492); the adaptive budget 512/1024/4096 moved one doubling per
step by decode pressure (:419-443); preemption newest first, keeping at least one page, with
the preempted requests going to the front of the queue (:269-347).

Where this scheduler decides differently:
* A request is a token list ``prompt + outputs`` with ``num_computed`` tokens in the cache.
  Whatever is not computed yet is run in portions; the portion that reaches the end asks for
  logits and yields the next token. The reference never takes logits from a prompt portion and
  re-runs the last prompt token as a decode row (:382-400).
* Preemption cuts the cache, not the outputs: the tokens already generated are kept and their
  keys/values recomputed like a prompt (the reference drops generated tokens and regenerates).
* The limits on sequences and on tokens in a step are separate (the reference's
  ``max_batch`` caps both, so its budget never binds).

When pages run out:
* at admission the request waits; a running request is never preempted to admit another. What is
  reserved at admission is the prompt's pages (``reserve="prompt"``, the default, as the reference
  does) or, with ``reserve="portion"``, only those of its first portion: then more requests are
  admitted than the pool can hold prompts of, the pages of later portions are taken when the portion
  is scheduled, and a portion that finds none has newer requests preempted for it like a decode row
  (if none can give, it waits for a later step);
* when a running request needs one more page to decode, running requests newer than it give
  tail pages, newest first and just as many as needed, and are preempted (they return to the
  front of the queue and recompute what they gave; while they wait they may be asked for the
  pages they kept, before any running request is cut); an older request is never cut for a newer
  one: if the newer ones cannot give enough, the request itself is preempted and waits, keeping
  its pages, or, if it is the only one running, is finished with reason "aborted".
"""
from __future__ import annotations

import hashlib
import itertools
import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Union

from ..cache import CacheManager
from ..sampling.params import SamplingParams


class SeqState(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED = "finished"


@dataclass
class Sequence_:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    max_gen: int
    seed: int
    state: SeqState = SeqState.WAITING
    outputs: List[int] = field(default_factory=list)
    num_computed: int = 0              # tokens of prompt + outputs whose keys/values are stored
    finish_reason: Optional[str] = None
    num_preemptions: int = 0
    prefix_hit_tokens: int = 0
    arrival_time: float = 0.0
    first_token_time: Optional[float] = None
    token_times: List[float] = field(default_factory=list)
    finish_time: Optional[float] = None
    admit_order: int = -1
    prefix_chain: Optional[list] = None    # chained hashes of the prompt's whole pages, made once

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.outputs

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.outputs)

    @property
    def prefill_done(self) -> bool:
        """Everything but the newest token is in the cache: the next step is a decode step."""
        return self.num_computed >= self.num_tokens - 1 and len(self.outputs) > 0


@dataclass
class ScheduledItem:
    seq: Sequence_
    start: int                         # first token position of the portion
    count: int                         # tokens in the portion
    want_logits: bool                  # the portion reaches the end of what is known
    fed: bool = False                  # a decode row whose token the step before it draws: not on the host yet

    @property
    def tokens(self) -> List[int]:
        seq, a, b = self.seq, self.start, self.start + self.count
        n = len(seq.prompt)
        if b <= n:
            return seq.prompt[a:b]
        if a >= n:
            return seq.outputs[a - n:b - n]
        return seq.prompt[a:] + seq.outputs[:b - n]


class RequestRejected(ValueError):
    pass


def default_seed(request_id: Hashable) -> int:
    """The seed of a request that names none: a digest of its id, the same in every process (Python's own
    ``hash`` of a string changes from run to run)."""
    return int.from_bytes(hashlib.blake2b(repr(request_id).encode(), digest_size=4).digest(), "little") & 0x7FFFFFFF


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_model_len: int, max_gen_len: int,
                 token_budget: Union[int, str] = "adaptive", eos_token_ids: Sequence[int] = (),
                 clock=time.monotonic, reserve: str = "prompt"):
        self.cache = cache
        self.max_num_seqs = int(max_num_seqs)
        self.max_model_len = int(max_model_len)
        self.max_gen_len = int(max_gen_len)
        self.adaptive = token_budget == "adaptive"
        self.token_budget = 1024 if self.adaptive else int(token_budget)   # scheduler.h:105 starts at 1024
        if self.token_budget < 1:
            raise ValueError("the token budget must be at least 1")
        if reserve not in ("prompt", "portion"):
            raise ValueError(f"reserve must be 'prompt' or 'portion', got {reserve!r}")
        self.reserve = reserve
        self.eos_token_ids = set(int(t) for t in eos_token_ids)
        self.clock = clock
        self.waiting: Deque[Sequence_] = deque()
        self.running: List[Sequence_] = []            # admission order
        self.finished: List[Sequence_] = []
        self._ids = itertools.count()
        self._admissions = itertools.count()
        self.num_steps = 0
        self.num_preemptions = 0
        self.num_recomputed_tokens = 0        # tokens whose keys and values a preemption gave up

    # ---- requests ------------------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    req_id: Optional[Hashable] = None) -> Hashable:
        """Queue a request; raises RequestRejected when it can never run (the reference returns
        -1 for a prompt that leaves no room to generate, scheduler.cpp:99-104)."""
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise RequestRejected("the prompt is empty")
        if len(prompt) >= self.max_model_len:
            raise RequestRejected(f"prompt of {len(prompt)} tokens leaves no room to generate within "
                                  f"max_model_len {self.max_model_len}")
        pool_tokens = min(g.pool.num_pages for g in self.cache.groups) * self.cache.page_size \
            if self.cache.groups else None
        if pool_tokens is not None and len(prompt) + 1 > pool_tokens:
            raise RequestRejected(f"prompt of {len(prompt)} tokens does not fit the cache of {pool_tokens} tokens")
        want = params.max_tokens if params.max_tokens is not None else self.max_gen_len
        max_gen = max(1, min(want, self.max_model_len - len(prompt)))      # scheduler.cpp:107-109
        rid = req_id if req_id is not None else next(self._ids)
        while req_id is None and self._is_live(rid):          # a counter value that a caller's own id has taken
            rid = next(self._ids)
        if self._is_live(rid):
            raise RequestRejected(f"a request with the id {rid!r} is waiting or running")
        seed = params.seed if params.seed is not None else default_seed(rid)
        seq = Sequence_(id=rid, prompt=prompt, params=params, max_gen=max_gen, seed=seed,
                        arrival_time=self.clock())
        self.waiting.append(seq)
        return rid

    def _is_live(self, rid) -> bool:
        return any(q.id == rid for q in self.running) or any(q.id == rid for q in self.waiting)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step: decide ------------------------------------------------------------------
    def schedule(self) -> List[ScheduledItem]:
        self.num_steps += 1
        self._admit()
        items: List[ScheduledItem] = []
        # decode rows first (scheduler.cpp:382-401), oldest first
        for seq in list(self.running):
            if seq.state is not SeqState.RUNNING or not seq.prefill_done:
                continue
            if not self._page_for_decode(seq):
                continue
            items.append(ScheduledItem(seq, seq.num_computed, 1, True))
        decoding = {id(it.seq) for it in items}
        pending = [s for s in self.running if s.state is SeqState.RUNNING and id(s) not in decoding
                   and not s.prefill_done]
        self._portions(items, pending, {}, may_preempt=True)
        # a portion may have had a newer request preempted whose decode row stood in this step already
        return [it for it in items if it.seq.state is SeqState.RUNNING]

    def schedule_ahead(self, inflight: Sequence[ScheduledItem]) -> Optional[List[ScheduledItem]]:
        """The step that follows ``inflight`` (launched, its tokens not read yet), decided before those
        tokens are known. Every request whose logits the step in flight takes will have one more token,
        unless that token is its last by length: it gets a decode row whose token is still on the device
        (``ScheduledItem.fed``). Prompt portions go on where the step in flight leaves them, and waiting
        requests are admitted, as ``schedule`` would do it. None when a decode row lacks a page: making
        room is left to ``schedule``, after the tokens have arrived. A request that the unread token
        ends (end of sequence) has a row all the same; ``update`` drops it."""
        self._admit()
        flying = {id(it.seq): it for it in inflight}
        items: List[ScheduledItem] = []
        pending: List[Sequence_] = []
        for seq in self.running:
            if seq.state is not SeqState.RUNNING:
                continue
            it = flying.get(id(seq))
            computed = it.start + it.count if it is not None else seq.num_computed
            unread = it is not None and it.want_logits
            if unread:
                if len(seq.outputs) + 1 >= seq.max_gen:
                    continue                              # ends by length with the unread token
                row = ScheduledItem(seq, computed, 1, True, fed=True)
            elif computed >= seq.num_tokens - 1 and seq.outputs:
                row = ScheduledItem(seq, computed, 1, True)      # a decode row whose token is known
            else:
                pending.append(seq)
                continue
            if not self.cache.can_grow(seq.id, row.start + 1):
                return None                               # pages taken for earlier rows stay with their requests
            self.cache.grow(seq.id, row.start + 1)
            items.append(row)
        self._portions(items, pending, {id(s): flying[id(s)].start + flying[id(s)].count
                                        for s in pending if id(s) in flying})
        if not items:
            return None
        self.num_steps += 1
        return items

    def _portions(self, items: List[ScheduledItem], pending: List[Sequence_], computed: Dict[int, int],
                  may_preempt: bool = False) -> None:
        """Prompt portions in admission order under the token budget, behind the decode rows in ``items``.
        ``computed``: where a request's cache will stand when the step runs, if not at ``num_computed``.
        With ``reserve="portion"`` a portion's pages are taken here; one that lacks pages has newer requests
        preempted for it (``may_preempt``: not while a step is in flight, whose requests must keep their
        pages), is cut down to the pages it has, or waits for a later step."""
        if not pending:
            return
        self._move_budget(len(items))
        taken = 0
        for seq in pending:
            if taken >= self.token_budget:
                break
            if seq.state is not SeqState.RUNNING:      # preempted for an older request's portion a moment ago
                continue
            start = computed.get(id(seq), seq.num_computed)
            remaining = seq.num_tokens - start
            take = min(remaining, self.token_budget - taken)
            if self.reserve == "portion":
                take = self._pages_for_portion(seq, start, take, may_preempt)
                if take <= 0:
                    continue
            items.append(ScheduledItem(seq, start, take, take == remaining))
            taken += take

    def _pages_for_portion(self, seq: Sequence_, start: int, take: int, may_preempt: bool) -> int:
        """Take the pages for tokens [start, start + take) of ``seq``; returns how many of the tokens have a
        place (0: none, the portion waits)."""
        if self.cache.can_grow(seq.id, start + take):
            self.cache.grow(seq.id, start + take)
            return take
        if may_preempt:
            ok = True
            for g, m in enumerate(self.cache.pages_missing(seq.id, start + take)):
                short = m - self.cache.free_pages(g)
                if short > 0 and not self._preempt_for(g, short, seq):
                    ok = False
                    break
            if ok and self.cache.can_grow(seq.id, start + take):
                self.cache.grow(seq.id, start + take)
                return take
        # what the free pages and the pages it holds cover
        ps = self.cache.page_size
        held = min(len(self.cache.table(g, seq.id)) + self.cache.free_pages(g) for g in range(len(self.cache.groups)))
        fit = min(take, held * ps - start)
        if fit <= 0:
            if may_preempt and not any(s is not seq and s.state is SeqState.RUNNING for s in self.running):
                self._finish(seq, "aborted")             # alone, every other request's pages taken, and still no room
            return 0
        self.cache.grow(seq.id, start + fit)
        return fit

    def _move_budget(self, decode_backlog: int) -> None:
        if not self.adaptive:
            return
        pressure = decode_backlog / self.max_num_seqs if self.max_num_seqs else 0.0
        target = 512 if pressure >= 0.5 else (4096 if pressure < 0.25 else 1024)
        if target > self.token_budget:
            self.token_budget = min(target, self.token_budget * 2)
        elif target < self.token_budget:
            self.token_budget = max(target, self.token_budget // 2)
        self.token_budget = max(512, min(4096, self.token_budget))

    def _admit(self) -> None:
        """First come, first served from the head of the queue; stop at the first request that
        does not fit (preempted requests sit at the head and come back first)."""
        while self.waiting and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            if not self.cache.has(seq.id):
                if self.cache.slots.num_free == 0:
                    break
                if seq.prefix_chain is None:               # a request that waits at the head is hashed once
                    seq.prefix_chain = self.cache.chain_hashes(seq.prompt)
                pages = self.cache.match_prefix(seq.prompt, seq.prefix_chain)
                need = self.cache.blocks_for(self._reserved_length(seq, len(pages) * self.cache.page_size)) - len(pages)
                if any(need > self.cache.free_pages(g) - self._parked_among(pages, g)
                       for g in range(len(self.cache.groups))):
                    break
                seq.num_computed = self.cache.admit(seq.id, seq.prompt, seq.prefix_chain)
                seq.prefix_hit_tokens = seq.num_computed
            elif not self.cache.can_grow(seq.id, self._reserved_length(seq, seq.num_computed)):
                break
            self.cache.grow(seq.id, self._reserved_length(seq, seq.num_computed))
            self.waiting.popleft()
            seq.state = SeqState.RUNNING
            if seq.admit_order < 0:
                seq.admit_order = next(self._admissions)
            self.running.append(seq)
            self.running.sort(key=lambda s: s.admit_order)

    def _reserved_length(self, seq: Sequence_, computed: int) -> int:
        """Tokens whose pages a request must get to be admitted: all it has, or its first portion's."""
        if self.reserve == "portion":
            return min(seq.num_tokens, computed + self.token_budget)
        return seq.num_tokens

    def _parked_among(self, pages: List[int], g: int) -> int:
        """Matched prefix pages that are counted as free (parked) but will be taken back."""
        if g != 0 or not self.cache.prefix_reuse:
            return 0
        pool = self.cache.groups[0].pool
        return sum(1 for p in pages if pool.is_parked(p))

    def _page_for_decode(self, seq: Sequence_) -> bool:
        """Make room for one more token of ``seq``; newer requests give pages if needed."""
        new_len = seq.num_tokens
        if self.cache.can_grow(seq.id, new_len):
            self.cache.grow(seq.id, new_len)
            return True
        missing = self.cache.pages_missing(seq.id, new_len)
        for g, m in enumerate(missing):
            short = m - self.cache.free_pages(g)
            if short > 0 and not self._preempt_for(g, short, seq):
                if any(s is not seq for s in self.running):
                    self._preempt_self(seq)              # the newest waits for the older ones
                else:
                    self._finish(seq, "aborted")         # alone and still too large for the pool
                return False
        self.cache.grow(seq.id, new_len)
        return True

    def _preempt_self(self, seq: Sequence_) -> None:
        seq.state = SeqState.PREEMPTED
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(seq)
        self._requeue([seq])

    def _requeue(self, preempted: List[Sequence_]) -> None:
        """Preempted requests wait at the front of the queue, oldest first (scheduler.cpp:305-311)."""
        front = [s for s in self.waiting if s.state is SeqState.PREEMPTED] + list(preempted)
        rest = [s for s in self.waiting if s.state is not SeqState.PREEMPTED]
        self.waiting = deque(sorted(front, key=lambda s: s.admit_order) + rest)

    def _preempt_for(self, group: int, need: int, requester: Sequence_) -> bool:
        """Free ``need`` pages of ``group``: first from requests that are preempted already and
        wait (they may give all they hold), then from running requests newer than the requester,
        newest first, each keeping at least one page unless that frees too little. Nothing happens unless enough
        can be freed
        (scheduler.cpp:269-313, which also takes from older requests)."""
        pool = self.cache.groups[group].pool
        ps = self.cache.page_size
        all_or_nothing = self.cache.can_truncate_to(ps) == 0      # windows or state: nothing can be kept

        def gain_if_cut(s: Sequence_, keep_pages: int) -> int:
            t = self.cache.table(group, s.id)
            return sum(1 for p in t[keep_pages:] if p >= 0 and pool.refcount(p) == 1)

        waiting = [s for s in self.waiting if s.state is SeqState.PREEMPTED and self.cache.has(s.id)]
        waiting.sort(key=lambda s: s.admit_order, reverse=True)
        running = [s for s in reversed(self.running)
                   if s.admit_order > requester.admit_order and s.state is SeqState.RUNNING]
        # running requests keep their first page if that frees enough; if not, they give everything too (a
        # pool in which every newer request holds one page would otherwise leave the older one waiting for ever)
        for running_keep in (1, 0):
            plan = []
            got = 0
            for s, min_keep in [(s, 0) for s in waiting] + [(s, running_keep) for s in running]:
                if got >= need:
                    break
                n = len(self.cache.table(group, s.id))
                if all_or_nothing:
                    keep = 0
                else:
                    keep = max(n - 1, min_keep)
                    while keep > min_keep and gain_if_cut(s, keep) < need - got:
                        keep -= 1
                g = gain_if_cut(s, keep)
                if g > 0:
                    plan.append((s, keep))
                    got += g
            if got >= need:
                break
        if got < need:
            return False
        newly = []
        for s, keep in plan:
            new_len = self.cache.truncate(s.id, keep * ps)
            self.num_recomputed_tokens += max(0, s.num_computed - new_len)
            s.num_computed = min(s.num_computed, new_len)
            if s.state is SeqState.RUNNING:
                s.state = SeqState.PREEMPTED
                s.num_preemptions += 1
                self.num_preemptions += 1
                self.running.remove(s)
                newly.append(s)
        self._requeue(newly)
        return True

    # ---- one step: take the results ----------------------------------------------------------
    def update(self, items: Sequence[ScheduledItem], sampled: Dict[Hashable, int]) -> List[Sequence_]:
        """``sampled`` maps request id to the token drawn from its wanted logits. Returns the
        requests that finished in this step."""
        now = self.clock()
        done: List[Sequence_] = []
        for it in items:
            seq = it.seq
            if seq.state is not SeqState.RUNNING:
                continue
            seq.num_computed = it.start + it.count
            if it.start < len(seq.prompt) <= seq.num_computed:
                self.cache.remember_prefix(seq.id, seq.prompt, seq.prefix_chain)
            if not it.want_logits:
                continue
            tok = int(sampled[seq.id])
            seq.outputs.append(tok)
            seq.token_times.append(now)
            if seq.first_token_time is None:
                seq.first_token_time = now
            stop = (not seq.params.ignore_eos and tok in self.eos_token_ids) or tok in seq.params.stop_token_ids
            if stop:
                self._finish(seq, "eos")
            elif len(seq.outputs) >= seq.max_gen:
                self._finish(seq, "length")
            if seq.state is SeqState.FINISHED:
                done.append(seq)
        return done

    def _finish(self, seq: Sequence_, reason: str) -> None:
        seq.state = SeqState.FINISHED
        seq.finish_reason = reason
        seq.finish_time = self.clock()
        if seq in self.running:
            self.running.remove(seq)
        if self.cache.has(seq.id):
            self.cache.release(seq.id)
        self.finished.append(seq)

    def abort_all(self, reason: str = "aborted") -> None:
        """A step failed: retire every request (the reference's force_finish_all,
        scheduler.cpp:496-513)."""
        for seq in list(self.running) + list(self.waiting):
            self._finish(seq, reason)
        self.waiting.clear()
