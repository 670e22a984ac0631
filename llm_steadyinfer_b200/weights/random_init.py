"""Random weights from a configuration and a seed: matrices and embeddings with mean 0 and
standard deviation 0.02, norm weights 1 + 0.1 z. Every element is a function of (seed, tensor
name, index of the element) alone, made of 64-bit integer arithmetic and one multiplication, so
that the same values come out on the CPU and on a GPU, bit for bit, and a tensor's values do not
depend on which other tensors exist: z is the sum of twelve uniform draws minus six (variance
one, bell-shaped, no value beyond six), each draw 21 bits of a splitmix64 hash of the element's
counter. ``write_random_model`` writes a model folder (config.json, model.safetensors) that the
loader reads like any checkpoint; ``init_random`` fills a model on its device without touching
the disk (large shapes), with the values a written folder of the same seed would hold. The
reference has no such mode.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from ..config.base import ModelConfig, config_from_dict
from .loader import place
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


_CHUNK = 1 << 24                    # elements drawn at a time (bounds the temporaries)
_GAMMA = -7046029254386353131       # 0x9E3779B97F4A7C15 as a signed 64-bit number
_MUL1 = -4658895280553007687        # 0xBF58476D1CE4E5B9
_MUL2 = -7723592293110705685        # 0x94D049BB133111EB


def _mix64(z: torch.Tensor) -> torch.Tensor:
    """The splitmix64 finaliser on int64 tensors (products wrap; the shifts are made logical by masks)."""
    z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * _MUL1
    z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * _MUL2
    return z ^ ((z >> 31) & ((1 << 33) - 1))


def tensor_key(seed: int, name: str) -> int:
    """The 62-bit key of a tensor's stream of draws."""
    h = hashlib.blake2b(f"{int(seed)}:{name}".encode(), digest_size=8).digest()
    return int.from_bytes(h, "little") >> 2


def standard_draws(key: int, first: int, count: int, device) -> torch.Tensor:
    """float64 [count]: the draws of elements first .. first + count - 1 of the stream ``key``."""
    idx = torch.arange(first, first + count, dtype=torch.int64, device=device)
    total = torch.zeros(count, dtype=torch.int64, device=device)
    for j in range(4):                                   # four hashes of three 21-bit draws each
        z = _mix64((idx * 4 + j) * _GAMMA + key)
        total += z & 0x1FFFFF
        total += (z >> 21) & 0x1FFFFF
        total += (z >> 42) & 0x1FFFFF
    # sum of (k + 1/2) / 2^21 over twelve draws, minus six; every step is exact in float64
    return (total.to(torch.float64) + (6.0 - 6.0 * 2097152.0)) * (1.0 / 2097152.0)


def _draw(name: str, shape, is_norm: bool, seed: int, device, store_dtype: torch.dtype) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    out = torch.empty(n, dtype=store_dtype, device=device)
    key = tensor_key(seed, name)
    for a in range(0, n, _CHUNK):
        z = standard_draws(key, a, min(_CHUNK, n - a), device)
        z = 1.0 + NORM_STD * z if is_norm else MATRIX_STD * z      # float64, rounded once below
        out[a:a + z.numel()] = z.to(store_dtype)
    return out.view(tuple(shape))


def random_tensors(model, seed: int, store_dtype: torch.dtype, device="cpu") -> Dict[str, torch.Tensor]:
    out = {}
    for name, shape in sorted(model.weight_shapes().items()):
        out[name] = _draw(name, shape, model.keeps_dtype(name), seed, device, store_dtype)
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
        t = _draw(name, shape, model.keeps_dtype(name), seed, model.device, store_dtype)
        tensors[name] = place(t, model.keeps_dtype(name), model.dtype, model.device)
    model.load_weights(tensors)
