"""Rotary position encoding part: owns the inverse frequencies, which a mixer hands to the
kernel that rotates q and k. Pairing is rotate-half, frequency of pair i is
``theta^(-2i/rot_dim)`` (reference: src/source/op/kernels/cuda/rope_kernel.cu:37-49 builds the
table entry j = 2i from ``theta^(-j/head_size)``). The reference has no frequency scaling;
the "llama3" rule rescales by wavelength ``lambda = 2*pi/f``:
``lambda < orig/high`` keeps f, ``lambda > orig/low`` gives ``f/factor``, and between them
``s = (orig/lambda - low)/(high - low)``, ``f' = (1 - s) * f/factor + s * f``.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position


def rotary_inverse_frequencies(rot_dim: int, theta: float, scaling) -> torch.Tensor:
    """fp32 [rot_dim/2], computed in float64 on the host."""
    i = torch.arange(0, rot_dim, 2, dtype=torch.float64)
    f = 1.0 / (float(theta) ** (i / rot_dim))
    if scaling is not None:
        kind = scaling.get("rope_type")
        if kind != "llama3":
            raise ValueError(f"rotary: scaling rule {kind!r} is not supported")
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        orig = float(scaling["original_max_position_embeddings"])
        wavelen = 2.0 * math.pi / f
        smooth = (orig / wavelen - low) / (high - low)
        mid = (1.0 - smooth) * f / factor + smooth * f
        f = torch.where(wavelen < orig / high, f, torch.where(wavelen > orig / low, f / factor, mid))
    return f.to(torch.float32)


class Rotary(PositionEncoding):
    capturable = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.head_dim = int(params["head_dim"])
        self.rot_dim = int(params.get("rot_dim") or self.head_dim)
        if self.rot_dim % 2 or self.rot_dim > self.head_dim:
            raise ValueError(f"rotary: rot_dim {self.rot_dim} must be even and at most head_dim")
        self.inv_freq = rotary_inverse_frequencies(
            self.rot_dim, params["theta"], params.get("scaling")).to(device)

    def rotary(self):
        return self.inv_freq, self.rot_dim


register_position("rotary", Rotary)
