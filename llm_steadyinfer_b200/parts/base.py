"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from the ``params`` of its spec alone (sizes and constants); it does not
know which model or layer it sits in. Four kinds exist:

``Norm``              ``forward(resid, delta, out, rows=None)``: add ``delta`` into the fp32
                      residual stream and normalise it into ``out``.
``PositionEncoding``  gives a mixer what it needs to encode positions: ``rotary()`` returns
                      ``(inv_freq, rot_dim)`` for mixers that fuse the rotation, or None, in
                      which case the mixer calls ``apply(q, k, ctx)`` on unfused views.
``Mixer``             ``forward(x, ctx, cache) -> delta`` mixes token rows of a sequence. A mixer or
                      feed-forward that says ``adds_into_residual = True`` is also given ``resid=`` (the fp32
                      stream) and may add its result there itself and return None (its last product then does
                      the add in its epilogue). It
                      (``prepare(ctx, cache)`` may plan the step on the host first); it
                      declares the cache it needs (``cache_need()``: paged keys/values, with or
                      without a window) and per-request state of fixed size (``state_need()``).
``FeedForward``       ``forward(x, ctx) -> delta`` acts on each row alone.

Every part lists the checkpoint tensors it wants under its prefix (``weight_shapes()``) and
takes them with ``load_weights()``; it may fuse or re-lay them out there.

A part whose ``forward`` can be captured into a CUDA graph says so with ``capturable = True``.

Another part is added by subclassing and ``register_mixer`` / ``register_feed_forward`` /
``register_norm`` / ``register_position`` under a new kind name; a configuration class then
names that kind in its layer specs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class CacheNeed:
    """Paged keys and values of one layer: pages of [num_kv_heads, page_size, head_dim],
    one for keys and one for values. ``window`` None keeps every token; otherwise pages
    that lie wholly before ``position - window + 1`` are given back."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self) -> Tuple:
        return ("paged_kv", self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one tensor of ``shape`` and ``dtype`` per request
    slot, zeroed when a request is admitted."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    # True if ``forward`` reads nothing on the host that changes from step to step: whatever depends on
    # the step comes from device tensors of ``ctx`` or is planned in ``prepare``, and nothing waits for
    # the device. Only then may a decode step be captured into a CUDA graph and replayed; a model with a
    # part that says False (the default, which is always right) runs every step directly.
    capturable = False
    # True if ``forward`` takes ``resid=`` (the fp32 residual stream) and may add its result into it itself,
    # returning None instead of the delta (mixers and feed-forwards; the default keeps the plain contract)
    adds_into_residual = False

    def __init__(self, params: Dict[str, Any], dtype: torch.dtype, device: torch.device):
        self.params = dict(params)
        self.dtype = dtype
        self.device = device

    def weight_shapes(self) -> Dict[str, Tuple[int, ...]]:
        """Checkpoint tensors below this part's prefix: name -> shape."""
        return {}

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take the tensors named by ``weight_shapes`` (already on the device)."""

    def keeps_dtype(self, name: str) -> bool:
        """True for tensors that stay in the dtype they are stored in (vectors such as norm
        weights); matrices are converted to the compute dtype."""
        return False

    def streams_first(self, rows: int) -> Optional[torch.Tensor]:
        """The weights that ``forward`` on ``rows`` rows reads first, if it streams them from memory once
        (few rows); the launch before it may fetch them into L2 ahead. None: nothing to fetch ahead."""
        return None

    def kernel_files(self, page_size: int) -> Tuple[str, ...]:
        """Names of the CUDA sources (``csrc/<name>.cu``) this part launches, so that they can be compiled
        together before the first step; a part that names none has its kernels compiled when first used."""
        return ()


class Norm(Part):
    # True if ``forward`` takes ``ahead=tensor``: what the part after the norm streams first, which the
    # norm's launch may start fetching into L2 (only asked of norms that say so)
    takes_ahead = False

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor], out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError

    def normalize(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> None:
        """The norm alone, over the last dimension of ``x`` (2-D or 3-D, last dimension contiguous), in place by
        default: for a norm that is not on the residual stream (one that a mixer applies to its queries and keys,
        head by head, say). Kinds that have no such form leave this unimplemented."""
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary(self) -> Optional[Tuple[torch.Tensor, int]]:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:
        """Encode positions into q [T, H, hs] and k [T, KV, hs] views in place."""
        raise NotImplementedError


class Mixer(Part):
    def __init__(self, params, dtype, device, position: Optional[PositionEncoding] = None):
        super().__init__(params, dtype, device)
        self.position = position

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def prepare(self, ctx, cache) -> None:
        """Host-side planning for the step (optional): runs once per step before any layer's
        ``forward``, and again before each replay of a captured step."""

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


_MIXERS: Dict[str, Callable] = {}
_FEED_FORWARDS: Dict[str, Callable] = {}
_NORMS: Dict[str, Callable] = {}
_POSITIONS: Dict[str, Callable] = {}


def _register(table: Dict[str, Callable], what: str):
    def reg(kind: str, cls) -> None:
        table[kind] = cls
    reg.__doc__ = f"Register a {what} class under a kind name used by specs."
    return reg


def _lookup(table: Dict[str, Callable], what: str):
    def get(kind: str):
        if kind not in table:
            raise KeyError(f"{what} kind {kind!r} is not registered; registered: {sorted(table)}")
        return table[kind]
    return get


register_mixer = _register(_MIXERS, "mixer")
register_feed_forward = _register(_FEED_FORWARDS, "feed-forward")
register_norm = _register(_NORMS, "norm")
register_position = _register(_POSITIONS, "position encoding")
mixer_class = _lookup(_MIXERS, "mixer")
feed_forward_class = _lookup(_FEED_FORWARDS, "feed-forward")
norm_class = _lookup(_NORMS, "norm")
position_class = _lookup(_POSITIONS, "position encoding")
