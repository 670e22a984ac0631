"""Llama 3 dense decoder: typed configuration and its model description.

Block structure follows the reference's ``LLamaModel::forward_batch``
(src/source/model/llama3.cpp:996-1181): RMSNorm, q/k/v projections without bias,
rotate-half RoPE, causal grouped-query attention over the cache, output projection,
residual; RMSNorm, gate/up projections, SiLU(gate)*up, down projection, residual;
final RMSNorm and LM head (llama3.cpp:1185-1194), tied to the embedding when
``tie_word_embeddings`` is set.

Unlike the reference (theta forced to 5e5 at model.cpp:368, eps fixed to 1e-6 at
rmsnorm_kernel.cu:120, no rope scaling), every constant is read from config.json.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, List, Optional, Union

from ..config.base import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelConfig,
                           ModelSpec, NormSpec, PositionSpec, read_key, register_architecture)


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json; only rope_type "llama3" carries parameters."""
    rope_type: str
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_position_embeddings: int = 0


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    tie_word_embeddings: bool
    hidden_act: str
    attention_bias: bool
    mlp_bias: bool
    torch_dtype: str
    bos_token_id: Optional[int]
    eos_token_id: Union[None, int, List[int]]

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        hidden = read_key(d, "hidden_size", int, positive=True)
        heads = read_key(d, "num_attention_heads", int, positive=True)
        kv_heads = read_key(d, "num_key_value_heads", int, heads, positive=True)
        if "head_dim" not in d or d["head_dim"] is None:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: 'hidden_size' {hidden} is not a multiple of "
                    f"'num_attention_heads' {heads} and no 'head_dim' is given")
            head_dim = hidden // heads
        else:
            head_dim = read_key(d, "head_dim", int, positive=True)
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: 'num_attention_heads' {heads} is not a multiple of "
                f"'num_key_value_heads' {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"config.json: 'head_dim' {head_dim} must be even for rotary pairs")

        rs = d.get("rope_scaling")
        scaling: Optional[RopeScaling] = None
        if rs is not None:
            if not isinstance(rs, dict):
                raise ConfigError("config.json: key 'rope_scaling' must be an object or null")
            rtype = rs.get("rope_type", rs.get("type"))
            if rtype in (None, "default"):
                scaling = None
            elif rtype == "llama3":
                scaling = RopeScaling(
                    rope_type="llama3",
                    factor=read_key(rs, "factor", float, positive=True),
                    low_freq_factor=read_key(rs, "low_freq_factor", float, positive=True),
                    high_freq_factor=read_key(rs, "high_freq_factor", float, positive=True),
                    original_max_position_embeddings=read_key(
                        rs, "original_max_position_embeddings", int, positive=True))
                if scaling.high_freq_factor <= scaling.low_freq_factor:
                    raise ConfigError("config.json: rope_scaling 'high_freq_factor' must exceed "
                                      "'low_freq_factor'")
            else:
                raise ConfigError(
                    f"config.json: rope_scaling rope_type {rtype!r} is not supported "
                    f"(supported: 'default', 'llama3')")

        act = read_key(d, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: 'hidden_act' {act!r} is not supported (supported: 'silu')")
        if read_key(d, "attention_bias", bool, False):
            raise ConfigError("config.json: 'attention_bias' true is not supported")
        if read_key(d, "mlp_bias", bool, False):
            raise ConfigError("config.json: 'mlp_bias' true is not supported")

        eos = d.get("eos_token_id")
        if eos is not None and not isinstance(eos, int):
            if not (isinstance(eos, list) and all(isinstance(e, int) for e in eos)):
                raise ConfigError("config.json: 'eos_token_id' must be an integer or a list of integers")
        bos = d.get("bos_token_id")
        if bos is not None and not isinstance(bos, int):
            raise ConfigError("config.json: 'bos_token_id' must be an integer")

        return cls(
            hidden_size=hidden,
            intermediate_size=read_key(d, "intermediate_size", int, positive=True),
            num_hidden_layers=read_key(d, "num_hidden_layers", int, positive=True),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=read_key(d, "vocab_size", int, positive=True),
            max_position_embeddings=read_key(d, "max_position_embeddings", int, positive=True),
            rms_norm_eps=read_key(d, "rms_norm_eps", float, positive=True),
            rope_theta=read_key(d, "rope_theta", float, positive=True),
            rope_scaling=scaling,
            tie_word_embeddings=read_key(d, "tie_word_embeddings", bool, False),
            hidden_act=act,
            attention_bias=False,
            mlp_bias=False,
            torch_dtype=read_key(d, "torch_dtype", str, "bfloat16"),
            bos_token_id=bos,
            eos_token_id=eos,
        )

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "llama"
        if self.rope_scaling is None:
            d["rope_scaling"] = None
        return d

    def eos_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        if isinstance(self.eos_token_id, int):
            return [self.eos_token_id]
        return list(self.eos_token_id)

    def model_spec(self) -> ModelSpec:
        position = PositionSpec("rotary", {
            "head_dim": self.head_dim,
            "theta": self.rope_theta,
            "scaling": None if self.rope_scaling is None else asdict(self.rope_scaling),
        })
        mixer = MixerSpec("attention", {
            "hidden_size": self.hidden_size,
            "num_heads": self.num_attention_heads,
            "num_kv_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "scale": self.head_dim ** -0.5,      # paged_kernels.cu:135 uses 1/sqrt(head size)
            "window": None,
        }, position=position)
        ffn = FeedForwardSpec("gated_mlp", {
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "activation": self.hidden_act,
        })
        norm = NormSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        layers = [
            LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm,
                      weight_prefix=f"model.layers.{i}.")
            for i in range(self.num_hidden_layers)
        ]
        return ModelSpec(
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            layers=layers,
            order=list(range(self.num_hidden_layers)),
            final_norm=norm,
            tie_word_embeddings=self.tie_word_embeddings,
            max_position=self.max_position_embeddings,
        )


register_architecture(LlamaConfig.architecture, LlamaConfig)
