"""Attention mixer: grouped-query causal attention over the paged cache, optional window.

Per row: q, k, v from one stacked projection [ (H + 2 KV) * hs, d ] (the reference stacks
them too, src/source/model/llama3.cpp:434-498, but then reads the output with the wrong row
stride, llama3.cpp:1009-1019; every consumer here takes the row stride); rotation of q and k
and the store of k, v into the sequence's pages; softmax(scale * q . K) V over cache
positions up to the row's own (llama3.cpp:1048-1067); output projection (llama3.cpp:1136-1140).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import CacheNeed, Mixer, register_mixer
from .linear import linear


class Attention(Mixer):
    def __init__(self, params, dtype, device, position=None):
        super().__init__(params, dtype, device, position)
        self.hidden = int(params["hidden_size"])
        self.H = int(params["num_heads"])
        self.KV = int(params["num_kv_heads"])
        self.hs = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = params.get("window") or None
        if self.H % self.KV:
            raise ValueError(f"attention: {self.H} heads are not a multiple of {self.KV} kv heads")
        if self.hs > 256:
            raise ValueError(f"attention: head_dim {self.hs} above 256 is not supported")
        self.qkv = None
        self.o = None

    def weight_shapes(self):
        return {"q_proj.weight": (self.H * self.hs, self.hidden),
                "k_proj.weight": (self.KV * self.hs, self.hidden),
                "v_proj.weight": (self.KV * self.hs, self.hidden),
                "o_proj.weight": (self.hidden, self.H * self.hs)}

    def load_weights(self, tensors):
        self.qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                              tensors["v_proj.weight"]], 0).contiguous()
        self.o = tensors["o_proj.weight"].contiguous()

    def cache_need(self):
        return CacheNeed(self.KV, self.hs, self.window)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        H, KV, hs = self.H, self.KV, self.hs
        qkv = ctx.buf("attn_qkv", (T, (H + 2 * KV) * hs), self.dtype)
        linear(x, self.qkv, qkv)
        rot = self.position.rotary() if self.position is not None else None
        if self.position is not None and rot is None:
            q3 = qkv[:, :H * hs].view(T, H, hs)
            k3 = qkv[:, H * hs:(H + KV) * hs].view(T, KV, hs)
            self.position.apply(q3, k3, ctx)
        inv_freq, rot_dim = rot if rot is not None else (None, 0)
        ops.rope_kv_write(qkv, ctx.positions, ctx.row_seq, inv_freq, rot_dim, cache.block_table,
                          cache.k if cache.writes else None, cache.v if cache.writes else None,
                          cache.page_size, ctx.num_seqs, H, KV, hs, status=ctx.status)
        attn = ctx.buf("attn_out", (T, H * hs), self.dtype)
        self.attend(qkv[:, :H * hs], cache, ctx, attn)
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(attn, self.o, out)
        return out

    def attend(self, q, cache, ctx, out):
        ops.paged_attention_ref(q, cache.k, cache.v, cache.block_table, ctx.row_seq, ctx.positions,
                                out, cache.page_size, ctx.num_seqs, self.H, self.KV, self.hs,
                                self.scale, self.window or 0, status=ctx.status)


register_mixer("attention", Attention)
