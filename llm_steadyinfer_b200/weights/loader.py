"""Weights by tensor name from a model folder (config.json + safetensors).

Matrices and embeddings are kept in the compute dtype (bfloat16 in the serving precision);
vectors that a part marks as dtype-keeping (norm weights) stay in the dtype they are stored
in when that is float32 or bfloat16, and integer tables are kept as int32. In the float32
precision everything floating is widened to float32. All faults of a checkpoint are reported
in one error: missing tensors, unexpected tensors and wrong shapes.
The reference instead slices an mmap by computed offsets and never checks a shape
(src/source/model/llama3.cpp:299-432).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch

from ..config.base import ModelConfig, load_config
from .safetensors_io import SafetensorsFile


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every fault."""


def checkpoint_files(model_dir: str) -> List[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map", {})
        files = sorted(set(wm.values()))
        return [os.path.join(model_dir, fn) for fn in files]
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    found = sorted(fn for fn in os.listdir(model_dir) if fn.endswith(".safetensors"))
    if not found:
        raise WeightError(f"no .safetensors file in {model_dir!r}")
    return [os.path.join(model_dir, fn) for fn in found]


def check_names_and_shapes(wanted: Dict[str, tuple], found: Dict[str, tuple], optional=()) -> None:
    missing = sorted(n for n in wanted if n not in found)
    unexpected = sorted(n for n in found if n not in wanted and n not in optional)
    wrong = sorted((n, wanted[n], found[n]) for n in wanted if n in found and tuple(found[n]) != tuple(wanted[n]))
    if not (missing or unexpected or wrong):
        return
    lines = ["checkpoint does not match the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + ", ".join(
            f"{n} expected {list(w)} found {list(f)}" for n, w, f in wrong))
    raise WeightError("\n".join(lines))


def place(t: torch.Tensor, keeps_dtype: bool, dtype: torch.dtype, device) -> torch.Tensor:
    """Move one stored tensor to the device in the dtype the engine keeps it in."""
    if not t.dtype.is_floating_point:
        return t.to(device=device, dtype=torch.int32)
    if dtype == torch.float32:
        target = torch.float32
    elif keeps_dtype and t.dtype in (torch.float32, torch.bfloat16):
        target = t.dtype
    else:
        target = dtype
    return t.to(device=device, dtype=target)


def load_weights_into(model, model_dir: str) -> None:
    files = [SafetensorsFile(p) for p in checkpoint_files(model_dir)]
    found: Dict[str, tuple] = {}
    where: Dict[str, SafetensorsFile] = {}
    for sf in files:
        for n in sf.names():
            found[n] = sf.shape(n)
            where[n] = sf
    wanted = model.weight_shapes()
    check_names_and_shapes(wanted, found, optional=model.optional_weights())
    tensors = {n: place(where[n].tensor(n), model.keeps_dtype(n), model.dtype, model.device)
               for n in wanted}
    model.load_weights(tensors)


def load_model(model_dir: str, dtype: torch.dtype, device="cuda:0"):
    """config.json picks the architecture; returns the model with its weights on the device."""
    from ..models import Model
    config: ModelConfig = load_config(model_dir)
    model = Model(config, dtype, device)
    load_weights_into(model, model_dir)
    return model
