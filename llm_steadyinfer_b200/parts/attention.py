"""Attention mixer: grouped-query causal attention over the paged cache, optional window.

Per row: q, k, v from one stacked projection [ (H + 2 KV) * hs, d ] (the reference stacks
them too, src/source/model/llama3.cpp:434-498, but then reads the output with the wrong row
stride, llama3.cpp:1009-1019; every consumer here takes the row stride); rotation of q and k
and the store of k, v into the sequence's pages; softmax(scale * q . K) V over cache
positions up to the row's own (llama3.cpp:1048-1067); output projection (llama3.cpp:1136-1140).
"""
from __future__ import annotations

import numpy as np
import torch

from ..csrc import ops
from .base import CacheNeed, Mixer, register_mixer
from . import linear as linear_mod
from .linear import linear


USE_TENSOR_CORES = True      # bf16 only; False sends bf16 through the plain kernel as well
USE_TMA = True               # decode tiles by TMA where the layout allows
USE_TC05 = True              # prompt portions on tcgen05 where the layout allows
FUSE_ROPE = True             # few rows (decode): rotation and cache store in the epilogue of the q/k/v product
DECODE_BLOCKS_PER_SM = 2     # decode attention blocks that one multiprocessor holds at once
MAX_SPLITS = 32
MIN_TILES_PER_SPLIT = 2      # a split covers at least this many 64-key tiles


class Attention(Mixer):
    adds_into_residual = True

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

    @property
    def capturable(self):
        """The step's work lists are made in ``prepare``; a position encoding applied through its
        unfused hook decides for itself."""
        return self.position is None or self.position.capturable

    def streams_first(self, rows):
        # few rows in bfloat16 go to the weight-streaming product, which reads every weight once
        return self.qkv if self.dtype == torch.bfloat16 and rows <= ops.SKINNY_MAX_ROWS else None

    def kernel_files(self, page_size):
        names = ["rope_kv"] + (["gemm_f32"] if self.dtype == torch.float32 else ["gemm_skinny", "gemm_rows", "gemm_tc05"])
        if not self.uses_tensor_cores():
            return tuple(names + ["attention_ref"])
        names.append("attention_mma")
        if self.hs in (64, 128) and page_size in (8, 16, 32, 64):        # the layouts the TMA-fed kernels take
            names += ["attention_tma"] * bool(USE_TMA) + ["attention_tc05"] * bool(USE_TC05)
        return tuple(names)

    def forward(self, x, ctx, cache, resid=None):
        T = x.shape[0]
        H, KV, hs = self.H, self.KV, self.hs
        qkv = ctx.buf("attn_qkv", (T, (H + 2 * KV) * hs), self.dtype)
        rot = self.position.rotary() if self.position is not None else None
        if (FUSE_ROPE and linear_mod.USE_SKINNY and rot is not None and rot[1] == hs and hs % 16 == 0
                and self.dtype == torch.bfloat16 and ops.gemm_skinny_ok(x, self.qkv, qkv)):
            # a decode step: one kernel for the projection, the rotation and the store into the pages
            ops.gemm_skinny_qkv_rope(x, self.qkv, qkv, ctx.positions, ctx.row_seq, rot[0], cache.block_table,
                                     cache.k if cache.writes else None, cache.v if cache.writes else None,
                                     cache.page_size, ctx.seq_slots, H, KV, hs, status=ctx.status)
            attn = ctx.buf("attn_out", (T, H * hs), self.dtype)
            self.attend(qkv[:, :H * hs], cache, ctx, attn)
            out = ctx.buf("delta", (T, self.hidden), self.dtype)
            linear(attn, self.o, out, ctx.status)
            return out
        linear(x, self.qkv, qkv, ctx.status)
        if self.position is not None and rot is None:
            q3 = qkv[:, :H * hs].view(T, H, hs)
            k3 = qkv[:, H * hs:(H + KV) * hs].view(T, KV, hs)
            self.position.apply(q3, k3, ctx)
        inv_freq, rot_dim = rot if rot is not None else (None, 0)
        ops.rope_kv_write(qkv, ctx.positions, ctx.row_seq, inv_freq, rot_dim, cache.block_table,
                          cache.k if cache.writes else None, cache.v if cache.writes else None,
                          cache.page_size, ctx.seq_slots, H, KV, hs, status=ctx.status)
        attn = ctx.buf("attn_out", (T, H * hs), self.dtype)
        self.attend(qkv[:, :H * hs], cache, ctx, attn)
        if resid is not None and linear_mod.linear_into_residual(attn, self.o, resid, ctx.status):
            return None                                   # the output projection added itself into the stream
        out = ctx.buf("delta", (T, self.hidden), self.dtype)
        linear(attn, self.o, out, ctx.status)
        return out

    # ---- kernels ---------------------------------------------------------------------
    def target_blocks(self) -> int:
        """Decode attention blocks that run at once on this part's device."""
        return DECODE_BLOCKS_PER_SM * ops.sm_count(self.device)

    def uses_tensor_cores(self) -> bool:
        return self.dtype == torch.bfloat16 and USE_TENSOR_CORES and self.hs % 16 == 0

    def prepare(self, ctx, cache):
        """Cut the step's sequences into work items for the tensor-core kernels: runs of few
        tokens (decode rows) for the decode kernel, longer portions in runs of the portion
        kernel's item size. One plan serves every layer with the same head layout and window."""
        if not self.uses_tensor_cores():
            return
        key = ("attention", self.H, self.KV, self.hs, self.window)
        if key in ctx.plans or cache.k is None:
            return
        G = self.H // self.KV
        tma = USE_TMA and ops.attn_decode_tma_ok(self.H, self.KV, self.hs, cache.page_size)
        dec_rows = ops.attn_decode_tma_rows(self.H, self.KV) if tma else ops.attn_decode_rows(self.H, self.KV, self.hs)
        dec_tokens = dec_rows // G
        tc05 = USE_TC05 and ops.attn_portion_tc05_ok(self.H, self.KV, self.hs, cache.page_size)
        por_tokens = (ops.attn_portion_tc05_tokens(self.H, self.KV) if tc05
                      else ops.attn_portion_tokens(self.H, self.KV, self.hs))
        if por_tokens <= 0:
            raise ops.KernelError(f"attention: {G} query heads per kv head do not fit the tensor-core kernels")
        dec, por = [], []
        S = ctx.num_seqs
        qs, cl = ctx.h_q_start, ctx.h_ctx_len
        for s in range(S):
            row0, n = int(qs[s]), int(qs[s + 1] - qs[s])
            pos0 = int(cl[s]) - n
            if n <= dec_tokens:
                dec.append((s, row0, n, pos0))
            else:
                for b in range(0, n, por_tokens):
                    por.append((s, row0 + b, min(por_tokens, n - b), pos0 + b))
        plan = {"dec": None, "por": None, "nsplit": 1, "scratch": None, "tma": tma, "work": None,
                "dec_rows": max((d[2] for d in dec), default=0) * G,
                "tc05": tc05}
        n_dec = len(dec)
        if ctx.seq_cap is not None:                   # fixed shapes: pad with empty items
            dec += [(0, 0, 0, 0)] * (ctx.seq_cap - n_dec)
        if dec and tma:
            # Shares of about equal length for as many blocks as run at once (two per SM), so that a long
            # sequence beside short ones is cut into more of them; a second wave of blocks would wait.
            tiles = []
            for (_, _, n, pos0) in dec:
                first = max(0, pos0 - self.window + 1) // 64 * 64 if self.window else 0
                tiles.append(-(-(pos0 + n - first) // 64) if n > 0 else 0)
            # Entries: every item whole, the shares that run at once, and room for finer cuts when items outnumber
            # those (entries without work are blocks that start and leave, so not more room than pays)
            budget = max(1, self.target_blocks() // self.KV)
            entries = budget + len(dec) + min(3 * len(dec), 2 * budget)
            work = ops.split_work(tiles, budget, entries, MAX_SPLITS, MIN_TILES_PER_SPLIT)
            if ctx.seq_cap is None:                    # shapes are free: only the entries with work
                work = work[:max(1, int((work[:, 0] >= 0).sum()))]
            both = ctx.upload_ints(f"attn_dec_{self.H}_{self.KV}_{self.hs}_{self.window}",
                                   np.concatenate([np.asarray(dec, dtype=np.int32).reshape(-1), work.reshape(-1)]))
            plan["dec"] = both[:4 * len(dec)].view(-1, 4)
            plan["work"] = both[4 * len(dec):].view(-1, 4)
            plan["scratch"] = ctx.buf("attn_split", (ops.attn_decode_tma_work_floats(entries, self.H, self.KV, self.hs),),
                                      torch.float32)
        elif dec:
            # as many blocks as run at once (two per SM), not more: a second wave would wait
            nsplit = max(1, min(MAX_SPLITS, self.target_blocks() // (len(dec) * self.KV)))
            if ctx.seq_cap is None:
                longest = max(d[3] + d[2] for d in dec)
                nsplit = min(nsplit, max(1, -(-longest // (64 * MIN_TILES_PER_SPLIT))))
            plan["nsplit"] = nsplit
            plan["dec"] = ctx.upload_ints(f"attn_dec_{self.H}_{self.KV}_{self.hs}_{self.window}",
                                          np.asarray(dec, dtype=np.int32)).view(-1, 4)
            if nsplit > 1:
                n = ops.attn_decode_scratch_floats(len(dec), self.H, self.KV, self.hs, nsplit)
                plan["scratch"] = ctx.buf("attn_split", (n,), torch.float32)
        if por:
            plan["por"] = ctx.upload_ints(f"attn_por_{self.H}_{self.KV}_{self.hs}_{self.window}",
                                          np.asarray(por, dtype=np.int32)).view(-1, 4)
        ctx.plans[key] = plan

    def attend(self, q, cache, ctx, out):
        if not self.uses_tensor_cores():
            ops.paged_attention_ref(q, cache.k, cache.v, cache.block_table, ctx.row_seq, ctx.positions,
                                    out, cache.page_size, ctx.seq_slots, self.H, self.KV, self.hs,
                                    self.scale, self.window or 0, status=ctx.status)
            return
        plan = ctx.plans[("attention", self.H, self.KV, self.hs, self.window)]
        args = (cache.page_size, ctx.seq_slots, self.H, self.KV, self.hs, self.scale, self.window or 0)
        if plan["dec"] is not None:
            if plan["tma"]:
                ops.attn_decode_tma(q, cache.k, cache.v, cache.block_table, plan["dec"], out, *args, work=plan["work"],
                                    scratch=plan["scratch"], status=ctx.status, max_rows=plan["dec_rows"])
            else:
                ops.attn_decode(q, cache.k, cache.v, cache.block_table, plan["dec"], out, *args,
                                nsplit=plan["nsplit"], scratch=plan["scratch"], status=ctx.status)
        if plan["por"] is not None:
            portion = ops.attn_portion_tc05 if plan["tc05"] else ops.attn_portion
            portion(q, cache.k, cache.v, cache.block_table, plan["por"], out, *args, status=ctx.status)


register_mixer("attention", Attention)
