"""A block arranges one mixer, one feed-forward and their norms around the residual stream.

How they are arranged is data as well: an *arrangement* is a function registered under a name,
``fn(block, resid, delta, ctx, cache) -> delta``, and a layer's spec names it. It gets the fp32
residual stream ``resid`` [T, d] and the pending ``delta`` of the block before it (None for the
first block), which it must add into the stream (``Norm.forward`` does the add and the norm in one
kernel), and returns its own pending delta, which the block after it (or the final norm) adds.

The built-in "pre_norm" is the reference's block (src/source/model/llama3.cpp:996-1181):
    h += delta_in;  x = norm1(h);  a = mixer(x);  h += a;  x = norm2(h);  return ffn(x)
Another arrangement (post-norm, parallel mixer and feed-forward, ...) is added with
``register_arrangement`` and needs no change here.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from .base import FeedForward, Mixer, Norm

_ARRANGEMENTS: Dict[str, Callable] = {}
_CAPTURABLE: Dict[str, bool] = {}


def register_arrangement(name: str, fn: Callable, capturable: bool = False) -> None:
    """Register ``fn(block, resid, delta, ctx, cache) -> delta`` under a name that layer specs use.
    ``capturable``: the function itself (beside the parts it calls) reads nothing on the host that
    changes from step to step, allocates nothing and never waits for the device, so that a decode
    step through it may be recorded in a CUDA graph (see ``Part.capturable``)."""
    _ARRANGEMENTS[name] = fn
    _CAPTURABLE[name] = bool(capturable)


def arrangement(name: str) -> Callable:
    if name not in _ARRANGEMENTS:
        raise KeyError(f"block arrangement {name!r} is not registered; registered: {sorted(_ARRANGEMENTS)}")
    return _ARRANGEMENTS[name]


class Block:
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm, arrangement_name: str = "pre_norm"):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.arrangement = arrangement_name
        self._run = arrangement(arrangement_name)
        self.capturable = _CAPTURABLE[arrangement_name]

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], ctx, cache) -> torch.Tensor:
        return self._run(self, resid, delta, ctx, cache)

    @staticmethod
    def norm(norm: Norm, resid, delta, out, ahead=None) -> None:
        """``resid += delta; out = norm(resid)``; ``ahead`` (what the part after the norm streams first)
        is passed on to norms that take it."""
        if ahead is not None and norm.takes_ahead:
            norm.forward(resid, delta, out, ahead=ahead)
        else:
            norm.forward(resid, delta, out)


def pre_norm(block: Block, resid, delta, ctx, cache):
    T, d = resid.shape
    x = ctx.buf("block_x", (T, d), block.mixer.dtype)
    block.norm(block.mixer_norm, resid, delta, x, block.mixer.streams_first(T))
    # a part that can add its result into the stream itself is given the stream and returns None
    if block.mixer.adds_into_residual:
        a = block.mixer.forward(x, ctx, cache, resid=resid)
    else:
        a = block.mixer.forward(x, ctx, cache)
    block.norm(block.feed_forward_norm, resid, a, x, block.feed_forward.streams_first(T))
    if block.feed_forward.adds_into_residual:
        return block.feed_forward.forward(x, ctx, resid=resid)
    return block.feed_forward.forward(x, ctx)


register_arrangement("pre_norm", pre_norm, capturable=True)
