"""Replay of given tokens through the step function, without sampling: the library side of
``bin/trace_run``. It owns nothing but the mapping from trace records to step entries; model,
cache and kernels are the engine's.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..weights import load_model
from .step import ModelRunner, StepEntry


class Replayer:
    def __init__(self, model_dir: str, dtype: torch.dtype, max_tokens: int, page_size: int = 16,
                 max_requests: int = 8, device: str = "cuda:0"):
        if 64 % page_size:
            raise ValueError(f"page size {page_size} must divide 64, the unit --max-tokens is counted in")
        model = load_model(model_dir, dtype, device)
        num_pages = max(1, -(-max_tokens // page_size))
        self.runner = ModelRunner(model, page_size=page_size, num_pages=num_pages,
                                  max_requests=max_requests, max_step_tokens=max(max_tokens, 64))

    def kept_after_truncate(self, held: int, keep: int) -> int:
        """Tokens a request of ``held`` tokens still holds after a ``truncate`` record with ``keep``: whole
        pages only, and nothing at all for a model with windows or fixed-size state."""
        return min(self.runner.manager.can_truncate_to(keep), held // self.runner.page_size * self.runner.page_size)

    def run_step(self, entries: Sequence[dict], end: Sequence = (), truncate: Sequence[dict] = ()) -> Optional[torch.Tensor]:
        """One trace record; returns the wanted logits on the host (fp32) or None. ``truncate``: records
        ``{"id": r, "keep": n}`` applied before the entries: request r is cut back to at most n tokens, as a
        preemption does (``kept_after_truncate`` says how many stay); the pages behind go back to the pool, and
        the trace feeds the cut tokens again."""
        out = None
        mgr = self.runner.manager
        for t in truncate:
            if not mgr.has(t["id"]):
                raise ValueError(f"truncate: request {t['id']!r} is not live")
            mgr.truncate(t["id"], int(t["keep"]))
        if entries:
            batch = [StepEntry(e["id"], list(e["tokens"]), list(e.get("want", ()))) for e in entries]
            logits = self.runner.step(batch)
            if logits is not None:
                out = logits.to("cpu")
            self.runner.check_status()
        for r in end:
            if self.runner.manager.has(r):
                self.runner.finish(r)
        return out
