"""Gated feed-forward part: ``down(silu(gate(x)) * up(x))`` without biases, as the reference's
block computes it (src/source/model/llama3.cpp:1149-1180). gate and up are stacked into one
[2F, d] matrix at load so one product feeds the activation: when F is a multiple of 8 the rows
are interleaved in groups of 8 (8 rows of gate, the 8 rows of up that belong to them, ...), so
that the few-row product holds a gate and its up in one block and applies the activation in
its epilogue. So does the product on the tcgen05 tensor cores for 128 rows and more (``gemm_tc05.cu``;
``gemm_rows.cu`` below that, when it is turned on); where none applies (fp32, an intermediate size that is
no multiple of 8, 17 to 127 rows by default), the product runs alone and the activation kernel reads the
same interleaved columns.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, register_feed_forward
from . import linear as linear_mod
from .linear import linear

INTERLEAVE = 8         # rows of gate, then rows of up, in the stacked weight
USE_TC05_GEMM = True   # gate/up product of more than 16 rows through this package's tcgen05 kernels (activation fused)


class GatedMLP(FeedForward):
    capturable = True
    adds_into_residual = True

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        if params.get("activation", "silu") != "silu":
            raise ValueError(f"gated_mlp: activation {params['activation']!r} is not supported")
        self.group = INTERLEAVE if self.inter % INTERLEAVE == 0 else self.inter
        self.gate_up = None
        self.down = None

    def weight_shapes(self):
        return {"gate_proj.weight": (self.inter, self.hidden),
                "up_proj.weight": (self.inter, self.hidden),
                "down_proj.weight": (self.hidden, self.inter)}

    def load_weights(self, tensors):
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        n = self.inter // self.group
        self.gate_up = torch.stack([gate.view(n, self.group, self.hidden), up.view(n, self.group, self.hidden)], 1) \
            .reshape(2 * self.inter, self.hidden).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def streams_first(self, rows):
        # few rows in bfloat16 go to the weight-streaming product, which reads every weight once
        return self.gate_up if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        if self.dtype == torch.float32:
            return ("gemm_f32", "swiglu")
        return ("gemm_skinny", "swiglu", "gemm_tc05", "gemm_rows")

    def forward(self, x, ctx, resid=None):
        T = x.shape[0]
        act = ctx.buf("ffn_act", (T, self.inter), self.dtype)
        if (self.group == INTERLEAVE and linear_mod.USE_SKINNY and act.dtype == torch.bfloat16
                and ops.gemm_skinny_ok(x, self.gate_up, act)):
            ops.gemm_skinny_swiglu(x, self.gate_up, act, checked=True)
        elif (self.group == INTERLEAVE and USE_TC05_GEMM and act.dtype == torch.bfloat16 and ops.gemm_tc05_available()
                and ops.gemm_tc05_ok(x, self.gate_up, act)
                and (linear_mod.USE_OWN_GEMM if T >= linear_mod.OWN_GEMM_MIN_ROWS else linear_mod.USE_ROWS)):
            if T >= linear_mod.OWN_GEMM_MIN_ROWS:
                ops.gemm_tc05_swiglu(x, self.gate_up, act, ctx.status)
            else:
                ops.gemm_rows_swiglu(x, self.gate_up, act, ctx.status)
        else:
            gu = ctx.buf("ffn_gate_up", (T, 2 * self.inter), self.dtype)
            linear(x, self.gate_up, gu, ctx.status)
            ops.swiglu(gu, act, self.group)
        if resid is not None and linear_mod.linear_into_residual(act, self.down, resid, ctx.status):
            return None                                   # the down projection added itself into the stream
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(act, self.down, out, ctx.status)
        return out


register_feed_forward("gated_mlp", GatedMLP)
