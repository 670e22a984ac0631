"""Configuration parsing and validation, the architecture registry, and the loader's errors."""
import json
import os

import pytest
import torch

from tiny_configs import TINY_A, TINY_B

from llm_steadyinfer_b200.config import ConfigError, config_from_dict, load_config, registered_architectures
from llm_steadyinfer_b200.models import Model
from llm_steadyinfer_b200.models.llama import LlamaConfig
from llm_steadyinfer_b200.weights import SafetensorsFile, WeightError, write_random_model, write_safetensors
from llm_steadyinfer_b200.weights.loader import check_names_and_shapes, load_weights_into


def test_registry_and_typed_fields():
    assert "LlamaForCausalLM" in registered_architectures()
    a = config_from_dict(TINY_A)
    b = config_from_dict(TINY_B)
    assert isinstance(a, LlamaConfig) and isinstance(b, LlamaConfig)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert a.rope_scaling is None and a.tie_word_embeddings and a.rms_norm_eps == 1e-5
    assert b.rope_scaling.factor == 8.0 and b.rope_scaling.original_max_position_embeddings == 64
    assert b.eos_token_ids() == [7, 9] and a.eos_token_ids() == [2]
    # defaults that derive from other keys
    d = dict(TINY_A); del d["head_dim"]; del d["num_key_value_heads"]
    c = config_from_dict(d)
    assert c.head_dim == 16 and c.num_key_value_heads == 4


def test_round_trip_through_json(tmp_path):
    for cfg in (TINY_A, TINY_B):
        c = config_from_dict(cfg)
        p = tmp_path / "m"
        p.mkdir(exist_ok=True)
        (p / "config.json").write_text(json.dumps(c.to_dict()))
        assert load_config(str(p)) == c


@pytest.mark.parametrize("change,needle", [
    ({"architectures": ["NoSuchModel"]}, "not registered"),
    ({"architectures": []}, "architectures"),
    ({"hidden_size": None}, "hidden_size"),
    ({"rms_norm_eps": "small"}, "rms_norm_eps"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"vocab_size": 10.5}, "vocab_size"),
])
def test_config_errors_name_the_key(change, needle):
    d = dict(TINY_A)
    d.update(change)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert needle in str(e.value)


def test_model_spec_is_data():
    spec = config_from_dict(TINY_B).model_spec()
    assert spec.order == [0, 1, 2] and len(spec.layers) == 3
    l0 = spec.layers[0]
    assert l0.mixer.kind == "attention" and l0.feed_forward.kind == "gated_mlp" and l0.mixer_norm.kind == "rmsnorm"
    assert l0.mixer.params["num_kv_heads"] == 1 and l0.mixer.position.kind == "rotary"
    assert l0.feed_forward.params["intermediate_size"] == 320 and l0.mixer_norm.params["eps"] == 1e-6


def test_weight_shapes_follow_the_config():
    m = Model(config_from_dict(TINY_B), torch.float32, "cpu")
    s = m.weight_shapes()
    assert s["model.embed_tokens.weight"] == (1000, 96) and s["lm_head.weight"] == (1000, 96)
    assert s["model.layers.2.self_attn.k_proj.weight"] == (32, 96)
    assert s["model.layers.0.mlp.down_proj.weight"] == (96, 320)
    assert s["model.norm.weight"] == (96,)
    tied = Model(config_from_dict(TINY_A), torch.float32, "cpu")
    assert "lm_head.weight" not in tied.weight_shapes()


def test_random_model_folder_is_seeded_and_bf16(tmp_path):
    write_random_model(str(tmp_path / "a"), TINY_A, 0)
    write_random_model(str(tmp_path / "b"), TINY_A, 0)
    write_random_model(str(tmp_path / "c"), TINY_A, 1)
    fa, fb, fc = (SafetensorsFile(str(tmp_path / x / "model.safetensors")) for x in "abc")
    names = sorted(fa.names())
    assert names == sorted(Model(config_from_dict(TINY_A), torch.float32, "cpu").weight_shapes())
    for n in names:
        assert fa.dtype(n) == torch.bfloat16
        assert torch.equal(fa.tensor(n), fb.tensor(n))
    assert not torch.equal(fa.tensor(names[0]), fc.tensor(names[0]))
    w = fa.tensor("model.layers.0.self_attn.q_proj.weight").float()
    g = fa.tensor("model.norm.weight").float()
    assert abs(w.std().item() - 0.02) < 0.003 and abs(g.mean().item() - 1.0) < 0.05
    assert load_config(str(tmp_path / "a")) == config_from_dict(TINY_A)
    # the safetensors library reads what the writer wrote
    from safetensors.torch import load_file
    lib = load_file(str(tmp_path / "a" / "model.safetensors"))
    assert all(torch.equal(lib[n], fa.tensor(n)) for n in names)


FIRST_DRAWS = [-0.44682979583740234, 0.6466436386108398, -0.1698441505432129]


def test_random_draws_are_a_function_of_seed_name_and_index():
    from llm_steadyinfer_b200.weights import random_init as ri
    key = ri.tensor_key(3, "model.layers.0.mlp.up_proj.weight")
    z = ri.standard_draws(key, 0, 1 << 18, "cpu")
    assert z.dtype == torch.float64
    # a draw depends on its index alone, not on where the chunk starts or how long it is
    assert torch.equal(ri.standard_draws(key, 1000, 77, "cpu"), z[1000:1077])
    assert abs(z.mean().item()) < 0.01 and abs(z.std().item() - 1.0) < 0.01 and z.abs().max().item() <= 6.0
    assert abs(((z ** 4).mean() / z.var() ** 2).item() - 2.9) < 0.05        # twelve uniforms: kurtosis 3 - 1/10
    assert abs(torch.corrcoef(torch.stack([z[:-1], z[1:]]))[0, 1].item()) < 0.01
    other = ri.standard_draws(ri.tensor_key(3, "model.layers.1.mlp.up_proj.weight"), 0, 1 << 18, "cpu")
    assert abs(torch.corrcoef(torch.stack([z, other]))[0, 1].item()) < 0.01
    assert ri.tensor_key(3, "a") != ri.tensor_key(4, "a") != ri.tensor_key(4, "b")
    # a tensor drawn in several chunks equals the same tensor drawn in one
    was = ri._CHUNK
    try:
        whole = ri._draw("w", (37, 29), False, 5, "cpu", torch.float32)
        ri._CHUNK = 100
        assert torch.equal(ri._draw("w", (37, 29), False, 5, "cpu", torch.float32), whole)
    finally:
        ri._CHUNK = was
    # fixed values: the draw is part of what a seed means, on every machine
    first = ri.standard_draws(ri.tensor_key(0, "model.embed_tokens.weight"), 0, 3, "cpu").tolist()
    assert first == pytest.approx(FIRST_DRAWS, abs=0)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = tmp_path / "m"
    write_random_model(str(d), TINY_A, 0)
    f = SafetensorsFile(str(d / "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    write_safetensors(str(d / "model.safetensors"), t)
    m = Model(load_config(str(d)), torch.float32, "cpu")
    with pytest.raises(WeightError) as e:
        load_weights_into(m, str(d))
    msg = str(e.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg and "missing" in msg
    assert "rotary_emb.inv_freq" in msg and "unexpected" in msg
    assert "k_proj.weight expected [32, 64] found [16, 64]" in msg


def test_tied_model_tolerates_a_stored_head_and_keeps_dtypes(tmp_path):
    d = tmp_path / "m"
    write_random_model(str(d), TINY_A, 0)
    f = SafetensorsFile(str(d / "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    t["model.norm.weight"] = t["model.norm.weight"].float()          # stored in 32-bit: stays so
    write_safetensors(str(d / "model.safetensors"), t)
    m = Model(load_config(str(d)), torch.bfloat16, "cpu")
    load_weights_into(m, str(d))
    assert m.final_norm.weight.dtype == torch.float32
    assert m.blocks[0].mixer_norm.weight.dtype == torch.bfloat16
    assert m.blocks[0].mixer.qkv.dtype == torch.bfloat16 and m.blocks[0].mixer.qkv.shape == (64 + 2 * 32, 64)
    assert m.lm_head is m.embed
    m32 = Model(load_config(str(d)), torch.float32, "cpu")
    load_weights_into(m32, str(d))
    assert m32.blocks[0].mixer.qkv.dtype == torch.float32 and m32.blocks[0].mixer_norm.weight.dtype == torch.float32


def test_shape_check_helper_alone():
    check_names_and_shapes({"a": (2, 3)}, {"a": (2, 3), "extra": (1,)}, optional=["extra"])
    with pytest.raises(WeightError):
        check_names_and_shapes({"a": (2, 3)}, {"a": (3, 2)})


def test_safetensors_rejects_a_torn_file(tmp_path):
    p = tmp_path / "x.safetensors"
    write_safetensors(str(p), {"a": torch.arange(6, dtype=torch.float32).view(2, 3), "n": torch.tensor([1, 2], dtype=torch.int64)})
    f = SafetensorsFile(str(p))
    assert f.tensor("a").tolist() == [[0, 1, 2], [3, 4, 5]] and f.dtype("n") == torch.int64
    raw = p.read_bytes()
    p.write_bytes(raw[:-4])
    with pytest.raises(ValueError):
        SafetensorsFile(str(p))


def test_no_cpu_fallback():
    """Kernels refuse CPU tensors instead of computing elsewhere."""
    from llm_steadyinfer_b200.csrc import ops
    with pytest.raises(ops.KernelError):
        ops.swiglu(torch.zeros(2, 8), torch.zeros(2, 4))
    from llm_steadyinfer_b200.parts.linear import linear
    with pytest.raises(ops.KernelError):
        linear(torch.zeros(2, 4), torch.zeros(3, 4), torch.zeros(2, 3))
