"""A block arranges one mixer, one feed-forward and their norms around the residual stream.

"pre_norm" (the reference's block, src/source/model/llama3.cpp:996-1181):
    h += delta_in;  x = norm1(h);  a = mixer(x);  h += a;  x = norm2(h);  return ffn(x)
Each residual add is fused into the norm that follows it, so a block takes the pending
``delta_in`` of the block before it and returns its own pending delta.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import FeedForward, Mixer, Norm

ARRANGEMENTS = ("pre_norm",)


class Block:
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm, arrangement: str = "pre_norm"):
        if arrangement not in ARRANGEMENTS:
            raise ValueError(f"block arrangement {arrangement!r} is not supported: {ARRANGEMENTS}")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.arrangement = arrangement

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx, cache) -> torch.Tensor:
        T, d = resid.shape
        x = ctx.buf("block_x", (T, d), self.mixer.dtype)
        self._norm(self.mixer_norm, resid, delta, x, self.mixer.streams_first(T))
        a = self.mixer.forward(x, ctx, cache)
        self._norm(self.feed_forward_norm, resid, a, x, self.feed_forward.streams_first(T))
        return self.feed_forward.forward(x, ctx)

    @staticmethod
    def _norm(norm: Norm, resid, delta, out, ahead) -> None:
        if ahead is not None and norm.takes_ahead:
            norm.forward(resid, delta, out, ahead=ahead)
        else:
            norm.forward(resid, delta, out)
