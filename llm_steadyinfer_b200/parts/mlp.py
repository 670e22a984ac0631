"""Gated feed-forward part: ``down(silu(gate(x)) * up(x))`` without biases, as the reference's
block computes it (src/source/model/llama3.cpp:1149-1180). gate and up are stacked into one
[2F, d] matrix at load so one product feeds the activation kernel.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, register_feed_forward
from .linear import linear


class GatedMLP(FeedForward):
    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        if params.get("activation", "silu") != "silu":
            raise ValueError(f"gated_mlp: activation {params['activation']!r} is not supported")
        self.gate_up = None
        self.down = None

    def weight_shapes(self):
        return {"gate_proj.weight": (self.inter, self.hidden),
                "up_proj.weight": (self.inter, self.hidden),
                "down_proj.weight": (self.hidden, self.inter)}

    def load_weights(self, tensors):
        self.gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], 0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, x, ctx):
        T = x.shape[0]
        gu = ctx.buf("ffn_gate_up", (T, 2 * self.inter), self.dtype)
        linear(x, self.gate_up, gu)
        act = ctx.buf("ffn_act", (T, self.inter), self.dtype)
        ops.swiglu(gu, act)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(act, self.down, out)
        return out


register_feed_forward("gated_mlp", GatedMLP)
