"""Typed model configuration: the base class, the architecture registry and the
specs that describe one model layer by layer.

A model is described as data:

* ``MixerSpec`` / ``FeedForwardSpec`` / ``NormSpec`` / ``PositionSpec`` name a
  registered part kind and carry its sizes and constants.
* ``LayerSpec`` puts one mixer, one feed-forward and their norms together and says
  which cache group the mixer stores into (or which other layer's cache it reads).
* ``ModelSpec`` holds the layer list and ``order``: the sequence in which layers run,
  which may name a layer twice.

The reference keeps a 36-byte binary header (src/include/model/config.h:4-31) and
derives sizes in ``Model::generate_model_infos`` (src/source/model/model.cpp:355-383);
here every size and constant comes from config.json keys.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type or an unsupported value."""


@dataclass(frozen=True)
class PositionSpec:
    kind: str                      # registered position-encoding kind, e.g. "rotary"
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class NormSpec:
    kind: str                      # e.g. "rmsnorm"
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class MixerSpec:
    kind: str                      # e.g. "attention"
    params: Dict[str, Any] = field(default_factory=dict)
    position: Optional[PositionSpec] = None


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                      # e.g. "gated_mlp"
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One block: ``h += mixer(norm(h)); h += ffn(norm(h))`` for arrangement "pre_norm".

    ``weight_prefix`` is the checkpoint prefix of this layer ("model.layers.3.").
    ``cache_from`` is None when the layer owns its cache, or the index of the layer
    whose cache it reads (it then writes nothing): that of the latest run of that layer
    before it in the run order.
    """
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    weight_prefix: str
    arrangement: str = "pre_norm"
    cache_from: Optional[int] = None
    # checkpoint names of the parts below weight_prefix
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_name: str = "input_layernorm."
    feed_forward_norm_name: str = "post_attention_layernorm."


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: List[LayerSpec]
    order: List[int]               # run order: indices into ``layers``
    final_norm: NormSpec
    tie_word_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm."
    lm_head_name: str = "lm_head.weight"
    max_position: int = 0


class ModelConfig:
    """Base of every architecture's typed configuration."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def model_spec(self) -> ModelSpec:
        raise NotImplementedError


_ARCHITECTURES: Dict[str, Callable[[Dict[str, Any]], ModelConfig]] = {}


def register_architecture(name: str, config_cls) -> None:
    """Map config.json's ``architectures[0]`` to a configuration class.

    The class's ``model_spec()`` is the architecture's model: the list of layers
    and the order they run in, built from registered parts.
    """
    _ARCHITECTURES[name] = config_cls


def registered_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def config_from_dict(d: Dict[str, Any]) -> ModelConfig:
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"config.json: architecture {name!r} is not registered; "
            f"registered: {registered_architectures()}")
    return _ARCHITECTURES[name].from_dict(d)


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)


# ---- helpers for typed reading -------------------------------------------------

_MISSING = object()


def read_key(d: Dict[str, Any], key: str, typ, default=_MISSING, *, positive=False):
    """Read ``d[key]`` as ``typ`` (int, float, bool, str); name the key on failure."""
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key {key!r} is missing")
        return default
    v = d[key]
    if typ is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if typ is int and isinstance(v, bool):
        raise ConfigError(f"config.json: key {key!r} must be an integer, found {v!r}")
    if not isinstance(v, typ):
        raise ConfigError(
            f"config.json: key {key!r} must be {typ.__name__}, found {type(v).__name__} {v!r}")
    if positive and not v > 0:
        raise ConfigError(f"config.json: key {key!r} must be positive, found {v!r}")
    return v
