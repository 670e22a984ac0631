"""The model: embedding, blocks in their run order, final norm and LM head, built from a
``ModelSpec`` with registered parts. It owns no cache and no batch logic: ``forward`` takes
the step's context (token rows, positions, block tables) and the per-layer cache views.

Data flow of the reference's ``forward_batch`` (src/source/model/llama3.cpp:849-1199), except
that the final norm and the LM head run on the wanted rows only (the reference computes
logits for every row of a mixed step and drops the prompt rows, scheduler.cpp:616-621).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..config.base import ModelConfig, ModelSpec
from ..csrc import ops
from ..parts import Block, feed_forward_class, mixer_class, norm_class, position_class
from ..parts.linear import configure_library_gemm, linear
from ..engine import tracing


class Model:
    def __init__(self, config: ModelConfig, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, found {dtype}")
        self.config = config
        self.spec: ModelSpec = config.model_spec()
        self.dtype = dtype
        self.device = torch.device(device)
        configure_library_gemm()
        self.blocks: List[Block] = []
        for ls in self.spec.layers:
            pos = None
            if ls.mixer.position is not None:
                pos = position_class(ls.mixer.position.kind)(ls.mixer.position.params, dtype, self.device)
            mixer = mixer_class(ls.mixer.kind)(ls.mixer.params, dtype, self.device, position=pos)
            ffn = feed_forward_class(ls.feed_forward.kind)(ls.feed_forward.params, dtype, self.device)
            n1 = norm_class(ls.mixer_norm.kind)(ls.mixer_norm.params, dtype, self.device)
            n2 = norm_class(ls.feed_forward_norm.kind)(ls.feed_forward_norm.params, dtype, self.device)
            self.blocks.append(Block(mixer, ffn, n1, n2, ls.arrangement))
        self.final_norm = norm_class(self.spec.final_norm.kind)(self.spec.final_norm.params, dtype, self.device)
        self.embed: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        for i in self.spec.order:
            if not 0 <= i < len(self.blocks):
                raise ValueError(f"run order names layer {i}, but the model has {len(self.blocks)} layers")

    # ---- weights -------------------------------------------------------------------
    def _named_parts(self):
        for ls, b in zip(self.spec.layers, self.blocks):
            p = ls.weight_prefix
            yield p + ls.mixer_prefix, b.mixer
            yield p + ls.feed_forward_prefix, b.feed_forward
            yield p + ls.mixer_norm_name, b.mixer_norm
            yield p + ls.feed_forward_norm_name, b.feed_forward_norm
        yield self.spec.final_norm_name, self.final_norm

    def weight_shapes(self) -> Dict[str, Tuple[int, ...]]:
        """Every checkpoint tensor the model wants: full name -> shape."""
        shapes = {self.spec.embed_name: (self.spec.vocab_size, self.spec.hidden_size)}
        if not self.spec.tie_word_embeddings:
            shapes[self.spec.lm_head_name] = (self.spec.vocab_size, self.spec.hidden_size)
        for prefix, part in self._named_parts():
            for n, s in part.weight_shapes().items():
                shapes[prefix + n] = tuple(s)
        return shapes

    def optional_weights(self) -> List[str]:
        """Tensors that may be in a checkpoint without being used (a stored head of a tied model)."""
        return [self.spec.lm_head_name] if self.spec.tie_word_embeddings else []

    def keeps_dtype(self, name: str) -> bool:
        for prefix, part in self._named_parts():
            if name.startswith(prefix) and name[len(prefix):] in part.weight_shapes():
                return part.keeps_dtype(name[len(prefix):])
        return False

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors`` holds every name of ``weight_shapes`` on the device, matrices in the
        compute dtype."""
        self.embed = tensors[self.spec.embed_name].contiguous()
        self.lm_head = self.embed if self.spec.tie_word_embeddings else tensors[self.spec.lm_head_name].contiguous()
        for prefix, part in self._named_parts():
            part.load_weights({n: tensors[prefix + n] for n in part.weight_shapes()})

    def kernel_files(self, page_size: int) -> List[str]:
        """CUDA sources of the model's own kernels and of its parts (see ``Part.kernel_files``)."""
        names = {"embedding", "sampling"} | ({"gemm_f32"} if self.dtype == torch.float32 else {"gemm_skinny", "gemm_rows", "gemm_tc05"})
        for _, part in self._named_parts():
            names.update(part.kernel_files(page_size))
        return sorted(names)

    def capturable(self) -> bool:
        """True if every part's ``forward`` may be captured into a CUDA graph (see ``Part.capturable``)."""
        return all(part.capturable for _, part in self._named_parts()) and all(b.capturable for b in self.blocks)

    # ---- forward -------------------------------------------------------------------
    def prepare(self, ctx, caches) -> None:
        """Host-side planning of the parts for this step (work lists, uploads); runs before
        ``forward`` and also before a captured step is replayed."""
        for o, i in enumerate(self.spec.order):
            self.blocks[i].mixer.prepare(ctx, caches[o])

    def forward(self, ctx, caches) -> Optional[torch.Tensor]:
        """Run the step's rows through all layers; returns fp32 logits [R, vocab] for
        ``ctx.logit_rows`` or None when no row is wanted. ``caches[o]`` is the view of the o-th
        place in the run order (a layer that runs twice has a cache per run)."""
        T, d = ctx.num_tokens, self.spec.hidden_size
        resid = ctx.buf("resid", (T, d), torch.float32)
        ops.embedding_gather(ctx.tokens, self.embed, resid, status=ctx.status)
        delta = None
        for o, i in enumerate(self.spec.order):
            if tracing.ENABLED:
                with tracing.span(f"layer {i}"):
                    delta = self.blocks[i].forward(resid, delta, ctx, caches[o])
            else:
                delta = self.blocks[i].forward(resid, delta, ctx, caches[o])
        R = ctx.num_logit_rows
        if R == 0:
            return None
        x = ctx.buf("final_x", (R, d), self.dtype)
        self.final_norm.forward(resid, delta, x, rows=ctx.logit_rows)
        logits = ctx.buf("logits", (R, self.spec.vocab_size), torch.float32)
        linear(x, self.lm_head, logits, ctx.status)
        return logits
