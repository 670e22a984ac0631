"""Runs the sampling kernel over the logits rows of a step: per-row temperature, top-k,
top-p, seed and the index of the output token travel in one pinned buffer; token ids come
back in one device-to-host copy."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device, max_rows: int):
        self.device = torch.device(device)
        self.max_rows = max_rows
        # per row: temperature f32, top_p f32, top_k i32, pad, seed i64, counter i64 -> 8 int32 words
        self._host = torch.empty(max_rows * 8, dtype=torch.int32, pin_memory=True)
        self._dev = torch.empty(max_rows * 8, dtype=torch.int32, device=self.device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=self.device)
        self._out_host = torch.empty(max_rows, dtype=torch.int32, pin_memory=True)
        self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
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
        h = self._host.numpy()
        n = self.max_rows
        h[0:R].view(np.float32)[:] = [p.temperature for p, _, _ in rows]
        h[n:n + R].view(np.float32)[:] = [p.top_p for p, _, _ in rows]
        h[2 * n:2 * n + R] = [p.top_k for p, _, _ in rows]
        h[4 * n:4 * n + 2 * R].view(np.uint64)[:] = [s & 0xFFFFFFFFFFFFFFFF for _, s, _ in rows]
        h[6 * n:6 * n + 2 * R].view(np.int64)[:] = [c for _, _, c in rows]
        self._dev.copy_(self._host, non_blocking=True)
        d = self._dev
        ops.sample(logits, out,
                   temperature=d[0:R].view(torch.float32), top_p=d[n:n + R].view(torch.float32),
                   top_k=d[2 * n:2 * n + R], seed=d[4 * n:4 * n + 2 * R].view(torch.int64),
                   counter=d[6 * n:6 * n + 2 * R].view(torch.int64))
        return out

    def to_host(self, tokens: torch.Tensor, status: torch.Tensor = None):
        """Device-to-host read of the sampled ids (synchronises the stream). With ``status`` (the
        engine's int32 status word) both travel before the one synchronisation and
        ``(ids, status code)`` is returned."""
        R = tokens.numel()
        self._out_host[:R].copy_(tokens, non_blocking=True)
        if status is not None:
            self._status_host.copy_(status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        ids = self._out_host[:R].tolist()
        return ids if status is None else (ids, int(self._status_host[0]))
