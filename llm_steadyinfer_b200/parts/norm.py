"""RMSNorm part: ``out = weight * h * rsqrt(mean(h^2) + eps)`` with ``h = resid + delta``
written back to the fp32 residual stream. Formula of the reference's
``row_rmsnorm_f32_dim`` (src/source/op/kernels/cuda/rmsnorm_kernel.cu:8-60), whose eps is a
constant in the kernel; here it is a parameter of the part.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import Norm, register_norm


class RMSNorm(Norm):
    capturable = True
    takes_ahead = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def weight_shapes(self):
        return {"weight": (self.size,)}

    def keeps_dtype(self, name: str) -> bool:
        return True

    def load_weights(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def kernel_files(self, page_size):
        return ("norm",)

    def forward(self, resid, delta, out, rows=None, ahead=None):
        ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, rows=rows, ahead=ahead)

    def normalize(self, x, out=None):
        ops.rmsnorm_rows(x, self.weight, self.eps, out)


register_norm("rmsnorm", RMSNorm)
