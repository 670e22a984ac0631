"""Tiny Llama 3 configurations that differ in every size and option (A and B; C sits at the layout
that the TMA and tcgen05 kernels take), and helpers that
write them as model folders with random weights into a temporary folder."""
import os

import torch

# heads 4 / kv 2 (grouped), head size 16, no frequency scaling, tied head
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "intermediate_size": 192, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "vocab_size": 512, "max_position_embeddings": 256, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "tie_word_embeddings": True,
    "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
    "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
}
# heads 3 / kv 1 (multi-query), head size 32, widths that are no power of two, llama3
# frequency scaling, untied head
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 96, "intermediate_size": 320, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "vocab_size": 1000, "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "tie_word_embeddings": False, "hidden_act": "silu", "attention_bias": False,
    "mlp_bias": False, "torch_dtype": "bfloat16", "bos_token_id": 0, "eos_token_id": [7, 9],
}
# head size 64 with grouped heads, pages of 16, an intermediate size that is a multiple of 8: the layout at
# which the TMA and tcgen05 kernels (decode attention, prompt attention, the gate/up product with the
# activation in its epilogue) take over from the general ones in bfloat16
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 256, "intermediate_size": 520, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "vocab_size": 777, "max_position_embeddings": 1024, "rms_norm_eps": 2e-6,
    "rope_theta": 100000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "tie_word_embeddings": False, "hidden_act": "silu", "attention_bias": False,
    "mlp_bias": False, "torch_dtype": "bfloat16", "bos_token_id": 0, "eos_token_id": 5,
}
CONFIGS = {"A": (TINY_A, 0, 16), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16)}     # config, seed, cache page size


def make_model_folder(tmp_path, name: str) -> str:
    from llm_steadyinfer_b200.weights import write_random_model
    cfg, seed, _ = CONFIGS[name]
    d = os.path.join(str(tmp_path), f"tiny_{name}")
    write_random_model(d, cfg, seed, torch.bfloat16)
    return d
