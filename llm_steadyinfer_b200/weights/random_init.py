"""Random weights from a configuration and a seed: matrices and embeddings ~ N(0, 0.02),
norm weights 1 + N(0, 0.1). Each tensor is drawn from a generator keyed by (seed, name), so
a tensor's values do not depend on which other tensors exist. ``write_random_model`` writes a
model folder (config.json, model.safetensors) that the loader reads like any checkpoint;
``init_random`` fills a model on its device without touching the disk (benchmarks of
large shapes). The reference has no such mode.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict

import torch

from ..config.base import ModelConfig, config_from_dict
from .loader import place
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _draw(name: str, shape, is_norm: bool, seed: int, device) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode())) % (2 ** 63))
    t = torch.randn(tuple(shape), generator=g, device=device, dtype=torch.float32)
    return 1.0 + NORM_STD * t if is_norm else MATRIX_STD * t


def random_tensors(model, seed: int, store_dtype: torch.dtype, device="cpu") -> Dict[str, torch.Tensor]:
    out = {}
    for name, shape in sorted(model.weight_shapes().items()):
        out[name] = _draw(name, shape, model.keeps_dtype(name), seed, device).to(store_dtype)
    return out


def write_random_model(model_dir: str, config, seed: int, store_dtype: torch.dtype = torch.bfloat16) -> None:
    """``config``: a ModelConfig or a config.json dictionary."""
    from ..models import Model
    cfg: ModelConfig = config if isinstance(config, ModelConfig) else config_from_dict(config)
    os.makedirs(model_dir, exist_ok=True)
    d = cfg.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                        torch.float16: "float16"}[store_dtype]
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=1)
    skeleton = Model(cfg, torch.float32, "cpu")
    write_safetensors(os.path.join(model_dir, "model.safetensors"),
                      random_tensors(skeleton, seed, store_dtype), metadata={"format": "pt", "seed": seed})


def init_random(model, seed: int, store_dtype: torch.dtype = torch.bfloat16) -> None:
    """Draw every tensor on the model's device, rounded through ``store_dtype`` as a written
    checkpoint would be."""
    tensors = {}
    for name, shape in sorted(model.weight_shapes().items()):
        t = _draw(name, shape, model.keeps_dtype(name), seed, model.device).to(store_dtype)
        tensors[name] = place(t, model.keeps_dtype(name), model.dtype, model.device)
    model.load_weights(tensors)
