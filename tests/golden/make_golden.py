"""Builds the reference's own Llama model code for its CPU device, runs it on two tiny random
models and stores what it computes, so that tests/plain_llama.py can be held against it.

    python tests/golden/make_golden.py --reference <root of the reference project>

Nothing of the reference is copied: its sources are compiled in place. The third-party headers
it expects (glog, armadillo, sentencepiece, re2) are replaced by the small stand-ins under
ref_build/shim, its tokenizer layer by ref_build/enc_stub.cpp, and ref_build/run_ref.cpp drives
``LLamaModel::forward_batch`` on a continuous cache and its ``Scheduler`` for greedy tokens.
The reference is run with LLAMA_DISABLE_FUSED_QKV=1, because its stacked-QKV path reads the
projection output with a wrong row stride (src/source/model/llama3.cpp:1009-1019), and with
block size = max sequence length, the only layout its CPU device supports.

The reference fixes theta = 5e5 (src/source/model/model.cpp:368), eps = 1e-6
(src/source/op/kernels/cpu/rmsnorm_kernel.cpp:56), has no frequency scaling and ties head size
to hidden/heads, so the two models use those values.

Outputs: golden_g1.npz, golden_g2.npz (weights, prompt, logits of every prompt position, and
greedy tokens of two requests), a few hundred KB together; golden_rope.npz (the reference's sine and
cosine tables at three values of theta, from its table function, which takes theta as an argument).
"""
import argparse
import glob
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = {
    "g1": dict(L=2, d=32, H=4, KV=2, F=48, V=64, tied=True, seed=0),
    "g2": dict(L=3, d=48, H=3, KV=1, F=80, V=100, tied=False, seed=1),
}
MAX_SEQ = 64
HOST_SOURCES = """base/base base/buffer base/alloc base/alloc_cpu base/alloc_cu tensor/tensor
op/layer op/matmul op/rmsnorm op/embedding op/add op/swiglu op/rope op/mha op/kernels/kernels_interfaces
op/kernels/cpu/add_kernel op/kernels/cpu/emb_kernel op/kernels/cpu/matmul_kernel op/kernels/cpu/mha_kernel
op/kernels/cpu/rmsnorm_kernel op/kernels/cpu/rope_kernel op/kernels/cpu/scale_kernel op/kernels/cpu/scale_sum_kernel
op/kernels/cpu/softmax_kernel op/kernels/cpu/swiglu_kernel model/model model/llama3 model/raw_model_data
scheduler/scheduler scheduler/kv_manager scheduler/block_allocator scheduler/prefix_cache
sampler/argmax_sampler""".split()
DEVICE_SOURCES = "add_kernel emb_kernel matmul_kernel mha_kernel paged_kernels rmsnorm_kernel rope_kernel swiglu_kernel argmax_kernel".split()


def build(ref: str, work: str) -> str:
    src = os.path.join(ref, "src")
    inc = ["-I", os.path.join(HERE, "ref_build", "shim"), "-I", os.path.join(src, "include"),
           "-I", "/usr/local/cuda/include", "-I", os.path.join(src, "source", "op", "kernels")]
    cxx = ["g++", "-std=c++17", "-O1", "-w", "-fopenmp", "-DUSE_PAGED_ATTENTION", "-include", "vector",
           "-include", "cstring", "-include", "fstream", "-include", "unistd.h"]
    objs = []
    jobs = []
    for s in HOST_SOURCES:
        o = os.path.join(work, s.replace("/", "_") + ".o")
        objs.append(o)
        jobs.append(cxx + inc + ["-c", os.path.join(src, "source", s + ".cpp"), "-o", o])
    for s in ("enc_stub", "run_ref"):
        o = os.path.join(work, s + ".o")
        objs.append(o)
        jobs.append(cxx + inc + ["-c", os.path.join(HERE, "ref_build", s + ".cpp"), "-o", o])
    for s in DEVICE_SOURCES:      # device objects only so that the link resolves; never executed
        o = os.path.join(work, "cu_" + s + ".o")
        objs.append(o)
        jobs.append(["nvcc", "-std=c++17", "-O1", "-w", "-arch=sm_90", "-DUSE_PAGED_ATTENTION", "-include", "vector",
                     "-include", "cstring"] + inc + ["-c", os.path.join(src, "source", "op", "kernels", "cuda", s + ".cu"), "-o", o])
    procs = []
    for j in jobs:
        procs.append(subprocess.Popen(j))
        if len(procs) >= 8:
            assert procs.pop(0).wait() == 0
    for p in procs:
        assert p.wait() == 0
    exe = os.path.join(work, "run_ref")
    subprocess.check_call(["nvcc", "-o", exe] + objs + ["-Xcompiler", "-fopenmp", "-lcublas", "-lgomp"])
    return exe


def make_case(name: str, c: dict, exe: str, work: str) -> None:
    L, d, H, KV, F, V = c["L"], c["d"], c["H"], c["KV"], c["F"], c["V"]
    hs = d // H
    kvd = KV * hs
    rng = np.random.default_rng(c["seed"])
    w = lambda *s: (rng.standard_normal(s) * 0.02).astype(np.float32)
    nw = lambda *s: (1 + rng.standard_normal(s) * 0.1).astype(np.float32)
    emb, an, wq, wk, wv, wo, fn = w(V, d), nw(L, d), w(L, H * hs, d), w(L, kvd, d), w(L, kvd, d), w(L, d, H * hs), nw(L, d)
    w1, w2, w3, fin = w(L, F, d), w(L, d, F), w(L, F, d), nw(d)
    cls = emb if c["tied"] else w(V, d)
    binp = os.path.join(work, name + ".bin")
    with open(binp, "wb") as f:      # header and tensor order of src/source/model/llama3.cpp:307-431
        f.write(struct.pack("8if", d, F, L, H, KV, (V if c["tied"] else -V), MAX_SEQ, 0, 500000.0))
        for a in (emb, an, wq, wk, wv, wo, fn, w1, w2, w3, fin):
            f.write(a.tobytes())
        f.write(np.zeros(MAX_SEQ * hs, np.float32).tobytes())
        if not c["tied"]:
            f.write(cls.tobytes())
    prompt = rng.integers(0, V, size=20)
    pp = os.path.join(work, name + ".prompt")
    with open(pp, "w") as f:
        f.write(" ".join(map(str, prompt)))
    lp = os.path.join(work, name + ".logits")
    env = dict(os.environ, SHIM_VOCAB=str(V), LLAMA_DISABLE_FUSED_QKV="1", LD_LIBRARY_PATH="/usr/local/cuda/lib64")
    out = subprocess.run([exe, binp, str(MAX_SEQ), pp, lp], env=env, capture_output=True, text=True, check=True).stdout
    gens = [[int(t) for t in line.split("gen:")[1].split()] for line in out.splitlines() if line.startswith("SEQ")]
    assert len(gens) == 2, out
    logits = np.fromfile(lp, np.float32).reshape(len(prompt), V)
    tensors = {"model.embed_tokens.weight": emb, "model.norm.weight": fin}
    if not c["tied"]:
        tensors["lm_head.weight"] = cls
    for l in range(L):
        p = f"model.layers.{l}."
        tensors.update({p + "input_layernorm.weight": an[l], p + "self_attn.q_proj.weight": wq[l],
                        p + "self_attn.k_proj.weight": wk[l], p + "self_attn.v_proj.weight": wv[l],
                        p + "self_attn.o_proj.weight": wo[l], p + "post_attention_layernorm.weight": fn[l],
                        p + "mlp.gate_proj.weight": w1[l], p + "mlp.down_proj.weight": w2[l],
                        p + "mlp.up_proj.weight": w3[l]})
    cfg = dict(hidden_size=d, intermediate_size=F, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=KV,
               vocab_size=V, rms_norm_eps=1e-6, rope_theta=500000.0, tie_word_embeddings=c["tied"])
    np.savez_compressed(os.path.join(HERE, f"golden_{name}.npz"), prompt=prompt.astype(np.int32), logits=logits,
                        gen_full=np.array(gens[0], np.int32), gen_short=np.array(gens[1], np.int32),
                        config=np.array(repr(cfg)), **{"w:" + k: v.astype(np.float16 if False else np.float32) for k, v in tensors.items()})
    print(name, "logits", logits.shape, "greedy", gens)


ROPE_CASES = [(16, 10000.0), (32, 500000.0), (64, 1000000.0)]      # (head size, theta); 96 positions each


def make_rope_tables(exe: str, work: str) -> None:
    """The reference's sine and cosine tables (src/source/op/kernels/cpu/rope_kernel.cpp:3-16) at three values of
    theta: its table function takes theta as an argument, so values other than the 5e5 of its model code are
    anchored on its code as well."""
    out = {}
    for hs, theta in ROPE_CASES:
        path = os.path.join(work, f"rope_{hs}.bin")
        subprocess.run([exe, "rope", str(hs), "96", repr(theta), path], check=True,
                       env=dict(os.environ, LD_LIBRARY_PATH="/usr/local/cuda/lib64"))
        t = np.fromfile(path, np.float32).reshape(2, 96, hs)
        out[f"sin_{hs}"], out[f"cos_{hs}"], out[f"theta_{hs}"] = t[0], t[1], np.float64(theta)
    np.savez_compressed(os.path.join(HERE, "golden_rope.npz"), **out)
    print("rope tables", sorted(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as work:
        exe = build(args.reference, work)
        for name, c in CASES.items():
            make_case(name, c, exe, work)
        make_rope_tables(exe, work)


if __name__ == "__main__":
    sys.exit(main())
