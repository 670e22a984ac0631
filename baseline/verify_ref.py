"""Checks the reference binary that bench.py's reference arm runs: its CUDA path (continuous KV layout) must
give the greedy tokens that its CPU path gave for the two tiny models of tests/golden.

    python baseline/verify_ref.py            (needs a GPU and baseline/_ref/ref_bench)

The weights, prompts and CPU tokens come from tests/golden/golden_g*.npz; the weights are written back into
the reference's .bin format (header and tensor order of src/source/model/llama3.cpp:307-431).
"""
import ast
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
MAX_SEQ = 64


def write_bin(path: str, g) -> int:
    cfg = ast.literal_eval(str(g["config"]))
    L, d, H, KV, F, V = (cfg["num_hidden_layers"], cfg["hidden_size"], cfg["num_attention_heads"],
                         cfg["num_key_value_heads"], cfg["intermediate_size"], cfg["vocab_size"])
    hs = d // H
    w = lambda n: g["w:" + n].astype("<f4")
    per = lambda n: np.stack([w(f"model.layers.{l}.{n}") for l in range(L)])
    tied = bool(cfg["tie_word_embeddings"])
    with open(path, "wb") as f:
        f.write(struct.pack("<8if", d, F, L, H, KV, (V if tied else -V), MAX_SEQ, 0, 500000.0))
        for a in (w("model.embed_tokens.weight"), per("input_layernorm.weight"), per("self_attn.q_proj.weight"),
                  per("self_attn.k_proj.weight"), per("self_attn.v_proj.weight"), per("self_attn.o_proj.weight"),
                  per("post_attention_layernorm.weight"), per("mlp.gate_proj.weight"), per("mlp.down_proj.weight"),
                  per("mlp.up_proj.weight"), w("model.norm.weight")):
            f.write(a.tobytes())
        f.write(np.zeros(MAX_SEQ * hs, "<f4").tobytes())
        if not tied:
            f.write(w("lm_head.weight").tobytes())
    return V


def main() -> int:
    exe = os.path.join(HERE, "_ref", "ref_bench")
    if not os.path.isfile(exe):
        print(f"{exe} is not built (python baseline/build_ref.py)")
        return 2
    ok = True
    with tempfile.TemporaryDirectory() as work:
        for name in ("g1", "g2"):
            g = np.load(os.path.join(ROOT, "tests", "golden", f"golden_{name}.npz"))
            binp, pp = os.path.join(work, name + ".bin"), os.path.join(work, name + ".prompt")
            V = write_bin(binp, g)
            with open(pp, "w") as f:
                f.write(" ".join(str(int(t)) for t in g["prompt"]))
            want = [g["gen_full"].tolist(), g["gen_short"].tolist()]
            # Its decode graphs: the first pure decode step of a batch size is recorded and never launched
            # (src/source/model/model.cpp:189-240 returns after cudaGraphInstantiate), so that step's token comes
            # from stale logits. With LLAMA_DISABLE_CUDA_GRAPH=1 (its own switch) every step runs.
            for graphs in (False, True):
                env = dict(os.environ, SHIM_VOCAB=str(V))
                if not graphs:
                    env["LLAMA_DISABLE_CUDA_GRAPH"] = "1"
                out = subprocess.run([exe, "verify", binp, str(MAX_SEQ), pp], env=env, capture_output=True, text=True, timeout=300)
                gens = [[int(t) for t in line.split("gen:")[1].split()] for line in out.stdout.splitlines() if line.startswith("SEQ")]
                same = out.returncode == 0 and gens == want
                if not graphs:
                    ok &= same
                print(f"{name}, decode graphs {'on' if graphs else 'off'}: reference on the GPU {gens}; on the CPU {want}: "
                      f"{'equal' if same else 'DIFFERENT'}"
                      + ("" if out.returncode == 0 else f" (exit {out.returncode}: {out.stdout[-200:]} {out.stderr[-200:]})"))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
