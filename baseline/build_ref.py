"""Builds the reference project's Llama engine, unmodified, into baseline/_ref/ref_bench for bench.py's
reference arm.

    python baseline/build_ref.py [--reference <root of the reference project>]

(default: $SI_REFERENCE_DIR, else the folder "reference" beside this repository)

The reference is a CMake/C++/CUDA project with no Python package, so ``pip install`` has nothing to install;
its sources are compiled in place here (nothing is copied or patched), with its CMake option
USE_PAGED_ATTENTION off: the continuous KV layout [layers, slots, kv_dim, max_seq_len] with its flash-decoding
kernels and three separate q/k/v products. (With the option on, its stacked-QKV path reads the projection
output with a wrong row stride, src/source/model/llama3.cpp:1009-1019, and its paged kernels give wrong
attention for more than one row; off, the GPU path gives the tokens its CPU path gives.) The third-party
headers the project expects (glog, armadillo, sentencepiece, re2) are not shipped with it; the stand-ins under
tests/golden/ref_build/shim replace them, and tests/golden/ref_build/enc_stub.cpp its tokenizer layer, which
the benchmark does not use (it feeds token ids). baseline/ref_bench.cpp is the driver.
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SHIM = os.path.join(ROOT, "tests", "golden", "ref_build")
OUT = os.path.join(HERE, "_ref")
HOST_SOURCES = """base/base base/buffer base/alloc base/alloc_cpu base/alloc_cu tensor/tensor
op/layer op/matmul op/rmsnorm op/embedding op/add op/swiglu op/rope op/mha op/kernels/kernels_interfaces
op/kernels/cpu/add_kernel op/kernels/cpu/emb_kernel op/kernels/cpu/matmul_kernel op/kernels/cpu/mha_kernel
op/kernels/cpu/rmsnorm_kernel op/kernels/cpu/rope_kernel op/kernels/cpu/scale_kernel op/kernels/cpu/scale_sum_kernel
op/kernels/cpu/softmax_kernel op/kernels/cpu/swiglu_kernel model/model model/llama3 model/raw_model_data
scheduler/scheduler scheduler/kv_manager scheduler/block_allocator scheduler/prefix_cache
sampler/argmax_sampler""".split()
DEVICE_SOURCES = "add_kernel emb_kernel matmul_kernel mha_kernel paged_kernels rmsnorm_kernel rope_kernel swiglu_kernel argmax_kernel".split()


def default_reference() -> str:
    return os.environ.get("SI_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")


def binary_path() -> str:
    return os.path.join(OUT, "ref_bench")


def build(reference: str, verbose: bool = True) -> str:
    src = os.path.join(reference, "src")
    if not os.path.isdir(os.path.join(src, "source", "model")):
        raise FileNotFoundError(f"no reference sources under {src}")
    work = os.path.join(OUT, "obj")
    os.makedirs(work, exist_ok=True)
    inc = ["-I", os.path.join(SHIM, "shim"), "-I", os.path.join(src, "include"), "-I", "/usr/local/cuda/include",
           "-I", os.path.join(src, "source", "op", "kernels")]
    pre = ["-include", "vector", "-include", "cstring", "-include", "fstream", "-include", "unistd.h"]
    cxx = ["g++", "-std=c++17", "-O2", "-w", "-fopenmp"] + pre
    nvcc = ["nvcc", "-std=c++17", "-O2", "-w", "-gencode", "arch=compute_100,code=sm_100", "-include", "vector", "-include", "cstring"]
    objs, jobs = [], []
    for s in HOST_SOURCES:
        o = os.path.join(work, s.replace("/", "_") + ".o")
        objs.append(o)
        jobs.append(cxx + inc + ["-c", os.path.join(src, "source", s + ".cpp"), "-o", o])
    for path in (os.path.join(SHIM, "enc_stub.cpp"), os.path.join(HERE, "ref_bench.cpp")):
        o = os.path.join(work, os.path.basename(path)[:-4] + ".o")
        objs.append(o)
        jobs.append(cxx + inc + ["-c", path, "-o", o])
    for s in DEVICE_SOURCES:
        o = os.path.join(work, "cu_" + s + ".o")
        objs.append(o)
        jobs.append(nvcc + inc + ["-c", os.path.join(src, "source", "op", "kernels", "cuda", s + ".cu"), "-o", o])
    procs = []
    for j in jobs:
        procs.append((j, subprocess.Popen(j)))
        if len(procs) >= 8:
            cmd, p = procs.pop(0)
            if p.wait() != 0:
                raise RuntimeError("failed: " + " ".join(cmd))
    for cmd, p in procs:
        if p.wait() != 0:
            raise RuntimeError("failed: " + " ".join(cmd))
    exe = binary_path()
    subprocess.check_call(["nvcc", "-o", exe] + objs + ["-Xcompiler", "-fopenmp", "-lcublas", "-lgomp",
                                                        "-Xlinker", "-rpath=/usr/local/cuda/lib64"])
    if verbose:
        print(f"built {exe}")
    return exe


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--reference", default=default_reference())
    args = ap.parse_args()
    build(args.reference)
    return 0


if __name__ == "__main__":
    sys.exit(main())
