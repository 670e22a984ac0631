"""The Python entry point: tokens in, tokens out.

``LLM`` puts the model, the step function, the scheduler and the sampler together in the manner
of the reference's drivers (benchmark/offline_batch_benchmark.cpp:199-300): requests are added
with ``add_request``, ``step()`` runs one scheduler step, ``all_finished()`` ends the loop and
``get_finished()`` hands the results back; ``generate`` wraps that loop. Option names follow the
reference's ``Scheduler(model, max_batch, max_seq_len, max_gen_len, block_size)``
(src/include/scheduler/scheduler.h:20-54).
"""
from __future__ import annotations

import collections
import time
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..sampling import Sampler, SamplingParams
from ..weights import load_model
from .scheduler import ScheduledItem, Scheduler, Sequence_
from . import tracing
from .step import ModelRunner, StepEntry


@dataclass
class GenerationResult:
    request_id: Hashable
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: Optional[str]
    num_preemptions: int = 0
    prefix_hit_tokens: int = 0


def _dtype_of(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
    if name not in table:
        raise ValueError(f"dtype must be one of {sorted(table)}, got {name!r}")
    return table[name]


class LLM:
    def __init__(self, model, dtype="bfloat16", max_batch: int = 32, max_seq_len: Optional[int] = None,
                 max_gen_len: int = 256, block_size: int = 16, num_blocks: Optional[int] = None,
                 max_num_batched_tokens: Union[int, str] = "adaptive", enable_prefix_cache: bool = True,
                 use_cuda_graph: bool = True, async_decode: bool = True, device: str = "cuda:0",
                 reserve: str = "prompt"):
        """``model``: a model folder or a built ``Model``. ``max_batch``: most requests running at
        once. ``max_seq_len``: most tokens (prompt + generated) of one request, by default the
        model's ``max_position``. ``num_blocks``: pages of the cache pool, by default
        ``max_batch * ceil(max_seq_len / block_size)`` as in the reference
        (src/source/scheduler/kv_manager.cpp:23-25). ``max_num_batched_tokens``: prompt tokens per
        step, or "adaptive" for the reference's 512/1024/4096 rule. ``async_decode``: while a
        step runs, the next one is already decided and launched (the tokens it draws pass to the
        next step on the device), so the host's work per step hides behind the GPU's. ``reserve``: pages
        a request must get to be admitted, its whole prompt's ("prompt", as the reference) or its first
        portion's ("portion": more requests run than the pool holds prompts of, and later portions preempt)."""
        self.dtype = _dtype_of(dtype)
        self.model = load_model(model, self.dtype, device) if isinstance(model, (str, bytes)) else model
        spec = self.model.spec
        self.max_seq_len = int(max_seq_len or spec.max_position)
        if spec.max_position and self.max_seq_len > spec.max_position:
            raise ValueError(f"max_seq_len {self.max_seq_len} exceeds the model's max_position {spec.max_position}")
        self.max_batch = int(max_batch)
        blocks_per_seq = -(-self.max_seq_len // block_size)
        self.num_blocks = int(num_blocks or self.max_batch * blocks_per_seq)
        budget_cap = 4096 if max_num_batched_tokens == "adaptive" else int(max_num_batched_tokens)
        self.runner = ModelRunner(self.model, page_size=block_size, num_pages=self.num_blocks,
                                  max_requests=self.max_batch, max_step_tokens=budget_cap + self.max_batch,
                                  prefix_reuse=enable_prefix_cache, max_seq_len=self.max_seq_len)
        eos = self.model.config.eos_token_ids() if hasattr(self.model.config, "eos_token_ids") else []
        self.scheduler = Scheduler(self.runner.manager, self.max_batch, self.max_seq_len, max_gen_len,
                                   token_budget=max_num_batched_tokens, eos_token_ids=eos, reserve=reserve)
        self.sampler = Sampler(self.model.device, self.max_batch)
        self.use_cuda_graph = bool(use_cuda_graph)
        self.async_decode = bool(async_decode)
        # steps are launched ahead only for models whose parts read nothing of a step on the host
        self._run_ahead = self.async_decode and self.runner.graphs_available()
        self._inflight = None             # a launched step whose tokens have not been read: (items, wanted, handle)
        self._returned = 0
        self._idle_steps = 0
        self.decode_host_ms = collections.deque(maxlen=1 << 16)    # host time of the latest steps that drew tokens
        self.stats = {"steps": 0, "decode_steps": 0, "graph_steps": 0, "ahead_steps": 0, "tokens_in": 0,
                      "tokens_out": 0, "steps_with_decode": 0}

    # ---- the reference's driver-facing calls ----------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        return self.scheduler.add_request(prompt_token_ids, params, request_id)

    def all_finished(self) -> bool:
        return self._inflight is None and not self.scheduler.has_unfinished()

    def get_running(self) -> List[Sequence_]:
        return list(self.scheduler.running)

    def get_finished(self) -> List[Sequence_]:
        """Requests finished since the last call."""
        out = self.scheduler.finished[self._returned:]
        self._returned = len(self.scheduler.finished)
        return out

    def step(self) -> List[Sequence_]:
        """One scheduler step: decide, run the model, sample, book the tokens. With ``async_decode`` a
        step is launched one call before its tokens are booked: the call launches the step after it as
        well, when that can be decided without the tokens (``Scheduler.schedule_ahead``), and only then
        waits for the tokens of the earlier one."""
        try:
            pending = self._inflight
            self._inflight = None
            if pending is None:
                with tracing.span("schedule"):
                    items = self.scheduler.schedule()
                if not items:
                    # nothing to run although requests are unfinished: a step or two may pass like this (requests
                    # requeued by a preemption are admitted by the next call), but never many
                    self._idle_steps += 1
                    if self._idle_steps > 8 and self.scheduler.has_unfinished():
                        raise RuntimeError(
                            f"the scheduler has found nothing to run for {self._idle_steps} steps although "
                            f"{len(self.scheduler.running)} running and {len(self.scheduler.waiting)} waiting "
                            f"requests are unfinished; they are aborted")
                    return []
                self._idle_steps = 0
                with tracing.span("launch"):
                    pending = self._launch(items)
            items, wanted, handle = pending
            if self._run_ahead:
                ahead = self.scheduler.schedule_ahead(items)
                if ahead is not None:
                    rows = {id(it.seq): r for r, it in enumerate(wanted)}
                    self._inflight = self._launch(ahead, src_rows=rows)
                    self.stats["ahead_steps"] += 1
            with tracing.span("resolve"):
                sampled = self._resolve(wanted, handle)
        except Exception:
            self._inflight = None
            self.scheduler.abort_all()
            raise
        self.stats["steps"] += 1
        return self.scheduler.update(items, sampled)

    def _launch(self, items: List[ScheduledItem], src_rows: Optional[Dict[int, int]] = None):
        """Queue one step on the GPU (model, sampling, copy of the ids to the host) without waiting for it.
        Rows with ``fed`` set take their token from the ids that the step before this one sampled, which
        are still on the device: ``src_rows`` maps ``id(request)`` to its row among that step's wanted rows."""
        t0 = time.perf_counter()
        entries = [StepEntry(it.seq.id, [0] if it.fed else it.tokens, [it.count - 1] if it.want_logits else [])
                   for it in items]
        feed = None
        if any(it.fed for it in items):
            dst, src, row = [], [], 0
            for it in items:
                if it.fed:
                    dst.append(row)
                    src.append(src_rows[id(it.seq)])
                row += it.count
            feed = (self.sampler.last_ids(), dst, src)
        pure_decode = all(it.count == 1 and it.want_logits for it in items)
        if pure_decode:
            self.stats["decode_steps"] += 1
        if pure_decode and self.use_cuda_graph and self.runner.graphs_available():
            logits = self.runner.step_decode_graph(entries, feed=feed)
            self.stats["graph_steps"] += 1
        else:
            logits = self.runner.step(entries, feed=feed)
        self.stats["tokens_in"] += sum(it.count for it in items)
        wanted = [it for it in items if it.want_logits]
        if wanted:
            # a step that draws tokens: the host's part of it (the batch's integers packed and copied, the launch),
            # which the reference's scheduler records for its decode steps as "batch reconstruct" time
            # (scheduler.cpp:560-573)
            self.stats["steps_with_decode"] += 1
            self.decode_host_ms.append((time.perf_counter() - t0) * 1e3)
        if not wanted:
            return items, wanted, None
        # the index of the output token keys the draw; a fed row draws the one after the unread token
        rows = [(it.seq.params, it.seq.seed, len(it.seq.outputs) + (1 if it.fed else 0)) for it in wanted]
        handle = self.sampler.fetch(self.sampler.sample(logits, rows), status=self.runner.status)
        return items, wanted, handle

    def _resolve(self, wanted: List[ScheduledItem], handle) -> Dict[Hashable, int]:
        if handle is None:
            self.runner.check_status()
            return {}
        tokens, code = self.sampler.wait(handle)
        self.runner.raise_status(code)
        self.stats["tokens_out"] += len(tokens)
        return {it.seq.id: t for it, t in zip(wanted, tokens)}

    # ---- convenience -------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[None, SamplingParams, Sequence[SamplingParams]] = None) -> List[GenerationResult]:
        """Run the prompts to the end; results in the order of ``prompts``."""
        if params is None or isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while not self.all_finished():
            self.step()
        by_id = {s.id: s for s in self.get_finished()}
        return [GenerationResult(i, by_id[i].prompt, by_id[i].outputs, by_id[i].finish_reason,
                                 by_id[i].num_preemptions, by_id[i].prefix_hit_tokens) for i in ids]
