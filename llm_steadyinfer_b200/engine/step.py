"""The step function: one batch of (request, its next tokens) through the model.

A step holds portions of prompts beside single decoded tokens, cut anywhere. It runs only the
tokens it is given, against what earlier steps left in the cache, and returns fp32 logits at
the wanted places. The reference's counterpart is ``forward_batch(input_ids, positions,
block_table, caches, logits, need_logits)`` (src/include/model/model.h:173-181); it uploads
one block-table row per *token* (src/source/scheduler/scheduler.cpp:526-551) and computes
logits for all rows, where this one uploads one row per *sequence* and a list of wanted rows.

All integer inputs of a step travel in one pinned buffer and one host-to-device copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import CacheLayout, CacheManager, CacheStorage, OutOfPages
from ..csrc.ops import KernelError

STATUS_TEXT = {
    1: "a token id is outside the vocabulary",
    2: "a block table entry is outside the page pool",
    3: "a row names a sequence outside the batch",
    4: "a bounded wait inside a kernel ran out",
}


@dataclass
class StepEntry:
    req: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are asked for


class StepError(RuntimeError):
    pass


class StepContext:
    """What every part sees of the running step."""

    def __init__(self, runner: "ModelRunner"):
        self._runner = runner
        self.num_tokens = 0
        self.num_seqs = 0
        self.num_logit_rows = 0
        self.status = runner.status
        self.plans: Dict = {}          # per-step scratch of parts (host-side plans), cleared each step
        # device int32 views, set by ModelRunner._stage
        self.tokens = self.positions = self.row_seq = None
        self.q_start = self.ctx_len = self.slots = self.logit_rows = None
        # host copies
        self.h_positions = self.h_q_start = self.h_ctx_len = self.h_slots = None
        self.seq_cap: Optional[int] = None   # set for fixed-shape decode steps (graphs): sequences the shapes are for

    def buf(self, key: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """A scratch tensor that lives until the same key is asked for again."""
        return self._runner.workspace(key, shape, dtype)

    def upload_ints(self, key: str, values: np.ndarray, capacity: Optional[int] = None) -> torch.Tensor:
        """Copy a small int32 array to a device buffer that keeps its address from step to step
        (parts send their per-step work lists through this from ``prepare``)."""
        return self._runner.upload_ints(key, values, capacity)


class ModelRunner:
    """Owns the model's cache (manager + storage), the step's staging buffers and scratch."""

    def __init__(self, model, page_size: int, num_pages: int, max_requests: int,
                 max_step_tokens: int, prefix_reuse: bool = False):
        if model.device.type != "cuda":
            raise KernelError("the engine runs on a CUDA device only; there is no CPU path")
        self.model = model
        self.device = model.device
        spec = model.spec
        self.layout = CacheLayout([b.mixer.cache_need() for b in model.blocks],
                                  [b.mixer.state_need() for b in model.blocks],
                                  [ls.cache_from for ls in spec.layers])
        self.manager = CacheManager(self.layout, page_size, num_pages, max_requests, prefix_reuse)
        self.storage = CacheStorage(self.layout, self.manager, model.dtype, self.device)
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_step_tokens = max_step_tokens
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._scratch: Dict[str, torch.Tensor] = {}
        self._stage_cap = 0
        self._hosts: List[torch.Tensor] = []      # ring of pinned buffers, one copy in flight each
        self._copied: List[Optional[torch.cuda.Event]] = []
        self._ring = 0
        self._dev = None
        self._uploads: Dict[str, dict] = {}
        self.ctx = StepContext(self)

    # ---- scratch -----------------------------------------------------------------------
    def workspace(self, key: str, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        k = (key, dtype)
        t = self._scratch.get(k)
        if t is None or t.numel() < n:
            if torch.cuda.is_current_stream_capturing():
                raise StepError(f"scratch {key!r} would have to grow during graph capture")
            t = torch.empty(max(n, 1), dtype=dtype, device=self.device)
            self._scratch[k] = t
        return t[:n].view(*shape)

    def upload_ints(self, key: str, values: np.ndarray, capacity: Optional[int] = None) -> torch.Tensor:
        values = np.ascontiguousarray(values, dtype=np.int32).reshape(-1)
        n = values.size
        cap = max(capacity or 0, n, 4)
        ent = self._uploads.get(key)
        if ent is None or ent["cap"] < cap:
            if torch.cuda.is_current_stream_capturing():
                raise StepError(f"upload buffer {key!r} would have to grow during graph capture")
            cap = max(cap, 2 * (ent["cap"] if ent else 0))
            ent = {"cap": cap, "ring": 0, "events": [None] * 4,
                   "hosts": [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(4)],
                   "dev": torch.empty(cap, dtype=torch.int32, device=self.device)}
            self._uploads[key] = ent
        ent["ring"] = (ent["ring"] + 1) % 4
        ev = ent["events"][ent["ring"]]
        if ev is not None:
            ev.synchronize()
        host = ent["hosts"][ent["ring"]]
        host.numpy()[:n] = values
        if n:
            ent["dev"][:n].copy_(host[:n], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            ent["events"][ent["ring"]] = ev
        return ent["dev"][:n]

    def _staging(self, n_ints: int):
        """A pinned host buffer whose last copy has finished, and the device buffer."""
        if n_ints > self._stage_cap:
            if torch.cuda.is_current_stream_capturing():
                raise StepError("staging buffers would have to grow during graph capture")
            torch.cuda.current_stream().synchronize()
            cap = max(1024, 2 * n_ints)
            self._hosts = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(4)]
            self._copied = [None] * 4
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._stage_cap = cap
        self._ring = (self._ring + 1) % len(self._hosts)
        ev = self._copied[self._ring]
        if ev is not None:
            ev.synchronize()
        return self._hosts[self._ring], self._dev

    def _upload(self, host: torch.Tensor, n_ints: int) -> None:
        self._dev[:n_ints].copy_(host[:n_ints], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._copied[self._ring] = ev

    # ---- the step ----------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one batch; returns fp32 logits [wanted rows, vocab] (a view into scratch that the
        next step overwrites) or None when nothing is wanted."""
        ctx = self._prepare(entries)
        self.storage.zero_new_slots()
        caches = self.storage.layer_views(self._tables)
        self.model.prepare(ctx, caches)
        logits = self.model.forward(ctx, caches)
        for e, new_len in zip(entries, self._new_lengths):
            self.manager.commit(e.req, new_len)
        return logits

    def _prepare(self, entries: Sequence[StepEntry], seq_cap: Optional[int] = None,
                 width_cap: Optional[int] = None) -> StepContext:
        mgr = self.manager
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        T = 0
        for e in entries:
            if e.req in seen:
                raise StepError(f"request {e.req!r} appears twice in one step")
            seen.add(e.req)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.req!r} brings no tokens")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"request {e.req!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
            T += len(e.tokens)
        if T > self.max_step_tokens:
            raise StepError(f"step of {T} tokens exceeds the limit of {self.max_step_tokens}")
        for e in entries:
            if not mgr.has(e.req):
                mgr.admit(e.req)
        # all-or-nothing over the whole step
        need = [0] * len(mgr.groups)
        for e in entries:
            for g, m in enumerate(mgr.pages_missing(e.req, mgr.length(e.req) + len(e.tokens))):
                need[g] += m
        for g, n in enumerate(need):
            if n > mgr.free_pages(g):
                raise OutOfPages(f"step needs {n} more pages in group {g}, {mgr.free_pages(g)} are free")
        self._new_lengths = []
        for e in entries:
            new_len = mgr.length(e.req) + len(e.tokens)
            mgr.grow(e.req, new_len)
            self._new_lengths.append(new_len)

        S = len(entries)
        R = sum(len(e.want) for e in entries)
        S_cap = seq_cap or S
        G = len(mgr.groups)
        W = max([1] + [len(mgr.table(g, e.req)) for g in range(G) for e in entries])   # pages may be reserved ahead
        W_cap = width_cap or W
        # layout (ints): tokens T | positions T | row_seq T | logit_rows R | q_start S+1 | ctx_len S | slots S | tables G*S*W
        offs = {}
        o = 0
        for name, n in (("tokens", T), ("positions", T), ("row_seq", T), ("logit_rows", max(R, 1)),
                        ("q_start", S_cap + 1), ("ctx_len", S_cap), ("slots", S_cap)):
            offs[name] = (o, n)
            o += (n + 3) // 4 * 4                     # 16-byte aligned regions
        table_off = o
        o += G * S_cap * W_cap
        host, dev = self._staging(o)
        h = host.numpy()
        row = 0
        r = 0
        b_tok, _ = offs["tokens"]; b_pos, _ = offs["positions"]; b_seq, _ = offs["row_seq"]
        b_lr, _ = offs["logit_rows"]; b_qs, _ = offs["q_start"]; b_cl, _ = offs["ctx_len"]; b_sl, _ = offs["slots"]
        h[b_qs:b_qs + S_cap + 1] = T
        h[b_cl:b_cl + S_cap] = 0
        h[b_sl:b_sl + S_cap] = 0
        for s, e in enumerate(entries):
            n = len(e.tokens)
            start = mgr.length(e.req)
            h[b_tok + row:b_tok + row + n] = np.asarray(e.tokens, dtype=np.int64).astype(np.int32)
            h[b_pos + row:b_pos + row + n] = np.arange(start, start + n, dtype=np.int32)
            h[b_seq + row:b_seq + row + n] = s
            h[b_qs + s] = row
            h[b_cl + s] = start + n
            h[b_sl + s] = mgr.slot(e.req)
            for w in e.want:
                h[b_lr + r] = row + w
                r += 1
            row += n
        tabs = h[table_off:table_off + G * S_cap * W_cap].reshape(G, S_cap, W_cap)
        tabs[:] = -1
        for g in range(G):
            for s, e in enumerate(entries):
                t = mgr.table(g, e.req)
                tabs[g, s, :len(t)] = t
        self._upload(host, o)

        ctx = self.ctx
        ctx.plans.clear()
        ctx.num_tokens, ctx.num_seqs, ctx.num_logit_rows = T, S, R
        view = lambda name, n: dev[offs[name][0]:offs[name][0] + n]
        ctx.tokens = view("tokens", T)
        ctx.positions = view("positions", T)
        ctx.row_seq = view("row_seq", T)
        ctx.logit_rows = view("logit_rows", R)
        ctx.q_start = view("q_start", S_cap + 1)
        ctx.ctx_len = view("ctx_len", S_cap)
        ctx.slots = view("slots", S_cap)
        ctx.h_positions = h[b_pos:b_pos + T].copy()
        ctx.h_q_start = h[b_qs:b_qs + S + 1].copy()
        ctx.h_ctx_len = h[b_cl:b_cl + S].copy()
        ctx.h_slots = h[b_sl:b_sl + S].copy()
        dtabs = dev[table_off:table_off + G * S_cap * W_cap].view(G, S_cap, W_cap)
        self._tables = [dtabs[g] for g in range(G)]
        return ctx

    def graphs_available(self) -> bool:
        return False

    def check_status(self) -> None:
        """Synchronise and raise if a kernel reported a fault (it never traps)."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise StepError(f"a kernel reported status {code}: {STATUS_TEXT.get(code, 'unknown')}")

    def finish(self, req: Hashable) -> None:
        """The request has ended; what it holds is given back."""
        self.manager.release(req)
