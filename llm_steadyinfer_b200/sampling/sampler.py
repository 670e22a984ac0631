"""Runs the sampling kernel over the logits rows of a step: per-row temperature, top-k,
top-p, seed and the index of the output token travel in one pinned buffer; token ids come
back in one device-to-host copy."""
from __future__ import annotations

from typing import Sequence, Tuple

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device, max_rows: int):
        self.device = torch.device(device)
        self.max_rows = max_rows
        # per row: temperature f32, top_p f32, top_k i32, pad, seed i64, counter i64 -> 8 int32 words
        # (four pinned copies in turn: with a step in flight the host already writes the next one's)
        self._hosts = [torch.empty(max_rows * 8, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._host_events = [None] * 4
        self._host_turn = 0
        self._dev = torch.empty(max_rows * 8, dtype=torch.int32, device=self.device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        # results: two pinned buffers (ids, then the status word), so that one step's ids can be read while
        # the next step's copy is already queued
        self._out_hosts = [torch.zeros(max_rows + 1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._out_turn = 0
        self._argmax_scratch = torch.zeros(ops.argmax_scratch_words(max_rows), dtype=torch.int32, device=self.device)

    def sample(self, logits: torch.Tensor, rows: Sequence[Tuple[SamplingParams, int, int]]) -> torch.Tensor:
        """``rows[r] = (params, seed, index of the output token)``; returns int32 [R] on the device."""
        R = logits.shape[0]
        if R != len(rows) or R > self.max_rows:
            raise ValueError(f"sampler got {R} logits rows for {len(rows)} requests (limit {self.max_rows})")
        out = self._out[:R]
        if all(p.greedy for p, _, _ in rows):
            ops.argmax(logits, out, self._argmax_scratch)
            return out
        self._host_turn = (self._host_turn + 1) % 4
        if self._host_events[self._host_turn] is not None:
            self._host_events[self._host_turn].synchronize()
        host = self._hosts[self._host_turn]
        h = host.numpy()
        n = self.max_rows
        h[0:R].view(np.float32)[:] = [p.temperature for p, _, _ in rows]
        h[n:n + R].view(np.float32)[:] = [p.top_p for p, _, _ in rows]
        h[2 * n:2 * n + R] = [p.top_k for p, _, _ in rows]
        h[4 * n:4 * n + 2 * R].view(np.uint64)[:] = [s & 0xFFFFFFFFFFFFFFFF for _, s, _ in rows]
        h[6 * n:6 * n + 2 * R].view(np.int64)[:] = [c for _, _, c in rows]
        self._dev.copy_(host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._host_events[self._host_turn] = ev
        d = self._dev
        ops.sample(logits, out,
                   temperature=d[0:R].view(torch.float32), top_p=d[n:n + R].view(torch.float32),
                   top_k=d[2 * n:2 * n + R], seed=d[4 * n:4 * n + 2 * R].view(torch.int64),
                   counter=d[6 * n:6 * n + 2 * R].view(torch.int64))
        return out

    def last_ids(self) -> torch.Tensor:
        """The device buffer that ``sample`` writes its ids into (valid until the next ``sample``)."""
        return self._out

    def fetch(self, tokens: torch.Tensor, status: torch.Tensor = None):
        """Queue the device-to-host copy of the sampled ids (and of the engine's int32 status word) and
        return a handle for ``wait``; the stream is not synchronised."""
        R = tokens.numel()
        self._out_turn ^= 1
        host = self._out_hosts[self._out_turn]
        host[:R].copy_(tokens, non_blocking=True)
        if status is not None:
            host[self.max_rows:self.max_rows + 1].copy_(status, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return (host, R, status is not None, ev)

    def wait(self, handle):
        """The ids of a ``fetch`` (and the status code when one was asked for), once its copy has arrived."""
        host, R, with_status, ev = handle
        ev.synchronize()
        ids = host[:R].tolist()
        return (ids, int(host[self.max_rows])) if with_status else ids

    def to_host(self, tokens: torch.Tensor, status: torch.Tensor = None):
        """Device-to-host read of the sampled ids. With ``status`` (the engine's int32 status word) both
        travel before the one wait and ``(ids, status code)`` is returned."""
        return self.wait(self.fetch(tokens, status))
