"""Per-request sampling options. The reference samples greedily only
(src/source/sampler/argmax_sampler.cpp:5-26) and bounds generation by ``max_gen_len`` and the
tokenizer's end-of-sentence id (src/source/scheduler/scheduler.cpp:655-694)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0          # 0 selects the greedy argmax
    top_p: float = 1.0
    top_k: int = 0                    # 0 keeps the whole vocabulary
    seed: Optional[int] = None        # None: derived from the request id
    max_tokens: Optional[int] = None  # None: the engine's max_gen_len
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError(f"max_tokens must be >= 1, got {self.max_tokens}")
        object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))

    @property
    def greedy(self) -> bool:
        return not self.temperature > 0
