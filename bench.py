"""Decode and prefill throughput of the engine at the Llama-3.1-8B shape, random weights, bf16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests whose contexts end at 8192 tokens.
``value`` is decoded tokens per second timed on the device around K steps (inputs staged from
pinned memory, CUDA-graph replay, sampling kernel; no host read inside the region); ``e2e`` is
the same through the Python entry point (``LLM.step``: scheduler, host-to-device copy of the
step's inputs, device-to-host read of the sampled tokens, every step). One JSON line is printed.
The engine runs on one GPU: for --gpus above 1 a line says so and the exit code is 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_3_1_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "hidden_act": "silu", "torch_dtype": "bfloat16",
    "bos_token_id": 128000, "eos_token_id": 128001,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}      # earlier measurement on this pool


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            pk = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"])}
            if isinstance(d.get("bf16_tflops_sustained"), (int, float)):
                pk["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])     # a long loop under the power cap
            return pk, "measured"
        except (ValueError, KeyError, TypeError, OSError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz = [int(r[0]) for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def write_reference_weights(path: str, cfg: dict, seq_len: int, layers: int) -> int:
    """A weights file in the reference's own format for the shape ``cfg``: the 36-byte header and raw fp32
    tensors in its grouped order (src/source/model/llama3.cpp:307-431), matrices ~ N(0, 0.02), norm weights 1.
    The values are one 64 MiB block of draws written over and over (the file is 32 GB at the 8B shape; timing
    does not depend on the values, only on their not being all alike). Returns the bytes written."""
    import struct
    import numpy as np
    d, F, H, KV, V = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"],
                      cfg["num_key_value_heads"], cfg["vocab_size"])
    hs = d // H
    L = layers
    rng = np.random.default_rng(0)
    tile = (rng.standard_normal(1 << 24) * 0.02).astype("<f4")
    ones = np.ones(1 << 20, dtype="<f4")
    total = 0
    with open(path, "wb", buffering=1 << 24) as f:
        f.write(struct.pack("<8if", d, F, L, H, KV, -V, seq_len, 0, float(cfg["rope_theta"])))   # negative: untied head
        total += 36

        def put(n, src):
            nonlocal total
            while n > 0:
                k = min(n, src.size)
                f.write(memoryview(src[:k]))
                n -= k
                total += 4 * k
        put(V * d, tile)                       # embedding
        put(L * d, ones)                       # attention norms
        put(L * H * hs * d, tile)              # wq
        put(L * KV * hs * d, tile)             # wk
        put(L * KV * hs * d, tile)             # wv
        put(L * d * H * hs, tile)              # wo
        put(L * d, ones)                       # feed-forward norms
        put(L * F * d, tile)                   # w1
        put(L * d * F, tile)                   # w2
        put(L * F * d, tile)                   # w3
        put(d, ones)                           # final norm
        put(seq_len * hs, ones)                # the skipped frequency tables
        put(V * d, tile)                       # output head
    return total


def reference_arm(args) -> int:
    """The same decode workload through the unmodified reference project: its binary (built by
    baseline/build_ref.py from the reference's sources, continuous KV layout) reads a random weights file of the
    same shape and runs ``Model::decode_step`` (device-timed ``value``) and ``Scheduler::step`` (``e2e``).
    Prints the JSON line of the contract with "impl": "reference", or why it is unavailable."""
    import shutil
    import tempfile

    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())}))
        return 0

    try:
        gpus = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=60)
        if gpus.returncode != 0 or "GPU 0" not in gpus.stdout:
            return unavailable("no CUDA device on this machine (nvidia-smi -L lists none)")
    except (OSError, subprocess.TimeoutExpired):
        return unavailable("no CUDA device on this machine (nvidia-smi cannot be run)")
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import build_ref
    except ImportError as e:
        return unavailable(f"baseline/build_ref.py cannot be imported: {e}")
    exe = build_ref.binary_path()
    if not os.path.isfile(exe):
        ref = build_ref.default_reference()
        if not os.path.isdir(ref):
            return unavailable("the reference is a CMake/C++ project without a Python package (pip has nothing to install); "
                               "its binary baseline/_ref/ref_bench has not been built and its sources are not on this machine")
        try:
            build_ref.build(ref, verbose=False)
        except Exception as e:      # noqa: BLE001
            return unavailable(f"building the reference failed: {e}")
    K, W = args.steps, max(3, args.warmup)
    B, CTX = args.batch, args.context
    cfg = dict(LLAMA_3_1_8B)
    L = args.layers or cfg["num_hidden_layers"]
    # The reference forms a tensor's size as a product of 32-bit ints (src/source/tensor/tensor.cpp:85): its cache
    # [layers, batch, kv_dim, context] must stay below 2^31 elements. At this shape and batch 8 that is a context
    # of 8,191, one token short of the bench's; it runs there.
    kv_dim = cfg["num_key_value_heads"] * (cfg["hidden_size"] // cfg["num_attention_heads"])
    CTX = min(CTX, ((1 << 31) - 1) // (L * B * kv_dim))
    d, F, V, H, KV = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hs = d // H
    floats = 2 * V * d + L * (2 * d + 2 * H * hs * d + 2 * KV * hs * d + 3 * F * d) + d + CTX * hs
    need = 4 * floats + 36
    folder = None
    for cand in (os.environ.get("TMPDIR"), tempfile.gettempdir(), "/dev/shm"):
        if cand and os.path.isdir(cand) and shutil.disk_usage(cand).free > need + (4 << 30):
            folder = tempfile.mkdtemp(prefix="si_ref_", dir=cand)
            break
    if folder is None:
        return unavailable(f"no temporary folder has room for the reference's {need >> 30} GB fp32 weights file")
    path = os.path.join(folder, "llama31_8b_shape.bin")
    rows = max(B, args.ref_rows)
    clocks = ClockSampler()
    try:
        write_reference_weights(path, cfg, CTX, L)
        env = dict(os.environ, SHIM_VOCAB=str(V))
        clocks.start()
        proc = subprocess.run([exe, "bench", path, str(B), str(CTX), str(K), str(W), str(rows), "1280"], env=env,
                              capture_output=True, text=True, timeout=1500)
        clocks.stop()
    except subprocess.TimeoutExpired:
        clocks.stop()
        return unavailable("the reference's run did not end within 25 minutes")
    except OSError as e:
        return unavailable(f"the reference's binary could not be run: {e}")
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    lines = [l for l in proc.stdout.strip().splitlines() if l.startswith("{")]
    if proc.returncode != 0 or not lines:
        return unavailable(f"the reference's run failed (exit {proc.returncode}): {lines[-1] if lines else ''}; "
                           f"its log ends: {proc.stderr[-400:]}")
    r = json.loads(lines[-1])
    if "error" in r:
        return unavailable(f"the reference's run failed: {r['error']}; its log ends: {proc.stderr[-400:]}")
    ms_per_step = r["device_ms"] / K
    out = {
        "metric": "decode tokens/s, Llama-3.1-8B shape, batch 8, context 8192", "value": round(B * K / r["device_ms"] * 1e3, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 (its stock dtype; products in TF32)",
        "data": "synthetic: random weights, random token ids", "impl": "reference",
        "config": {"model": "Llama-3.1-8B shape", "layers": L, "layers_full": cfg["num_hidden_layers"], "hidden": d, "heads": H,
                   "kv_heads": KV, "head_dim": hs, "intermediate": F, "vocab": V, "global_batch": B, "seq_len": CTX,
                   "parallelism": "single_gpu", "cuda_graph": True, "kv_layout": "continuous (USE_PAGED_ATTENTION off)",
                   "scheduler_rows": rows, "seq_len_note": "largest context its 32-bit tensor sizes hold at this batch"},
        "e2e": {"value": round(r["e2e_tokens"] / r["e2e_s"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": r["d2h_bytes_per_step"],
                "how": "Model::decode_step + post_processing_batch every step, as its Scheduler runs a decode step"},
        # 1,024-token prompts and 256 generated tokens through its own Scheduler, timed while all requests decode
        "points": {"decode_b8_ctx1280_scheduler": r["sched_tokens_per_s"], "decode_b8_ctx1280_scheduler_ms": r["sched_ms_per_step"],
                   "decode_b8_ctx1280_scheduler_mean_context": r.get("sched_mean_context")},
        "clocks": clocks.summary(),
    }
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--ref-rows", type=int, default=32,
                    help="--impl reference: rows a step of its scheduler (its max_batch_size, which also caps a prompt portion)")
    ap.add_argument("--profiler-range", action="store_true",
                    help="bracket the timed region of --section with cudaProfilerStart/Stop "
                         "(for ncu --profile-from-start off)")
    ap.add_argument("--section", default="all", choices=["all", "decode", "prefill"],
                    help="run only the device-timed decode steps or only the prefill (for profiling)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    K, W = args.steps, max(3, args.warmup)

    import torch
    from llm_steadyinfer_b200 import LLM, SamplingParams
    from llm_steadyinfer_b200.config import config_from_dict
    from llm_steadyinfer_b200.csrc import ops
    from llm_steadyinfer_b200.engine.step import StepEntry
    from llm_steadyinfer_b200.models import Model
    from llm_steadyinfer_b200.weights import init_random

    torch.cuda.set_device(0)
    cfg_d = dict(LLAMA_3_1_8B)
    layers_full = cfg_d["num_hidden_layers"]
    if args.layers:
        cfg_d["num_hidden_layers"] = args.layers
    cfg = config_from_dict(cfg_d)
    model = Model(cfg, torch.bfloat16, "cuda:0")
    init_random(model, seed=0)
    B, CTX, PAGE = args.batch, args.context, 16
    big = 1 if (args.no_points or args.section != "all") else max(B, 64)
    llm = LLM(model, dtype="bfloat16", max_batch=max(B, big), max_seq_len=CTX, max_gen_len=K + W + 16 + args.batch * (-(-args.context // 2048)),
              block_size=PAGE, max_num_batched_tokens=2048, enable_prefix_cache=False)
    runner, mgr = llm.runner, llm.runner.manager
    gen = torch.Generator().manual_seed(1)
    V = cfg.vocab_size
    rand_tokens = lambda n: torch.randint(0, V, (n,), generator=gen).tolist()
    pk, pk_src = peaks()
    L, d, F = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size
    H, KV, hs = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    block_params = L * (d * (H + 2 * KV) * hs + H * hs * d + 3 * d * F)
    weight_bytes = 2 * (block_params + V * d) + 2 * (2 * L + 1) * d
    kv_bytes_per_token = 2 * L * KV * hs * 2

    def timed(fn, n):
        torch.cuda.synchronize()
        if args.profiler_range:
            torch.cuda.cudart().cudaProfilerStart()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        if args.profiler_range:
            torch.cuda.cudart().cudaProfilerStop()
        return a.elapsed_time(b)

    clocks = ClockSampler()

    # ---- prefill of 2,048 tokens (one request, logits of the last row) -----------------------
    PT = 2048
    ptoks = rand_tokens(PT)

    def prefill_once(i):
        runner.step([StepEntry("prefill", ptoks, [PT - 1])])
        runner.finish("prefill")

    def kernel_time_shares():
        """Share of the summed kernel time per kind of kernel, for one prompt step of 2,048 tokens and one direct
        (not recorded) decode step of the bench's batch and context; events sit between the kernels, so these
        are shares, not the step's time."""
        from llm_steadyinfer_b200.engine.kernel_times import KernelTimes
        out = {}
        with KernelTimes() as kt:
            prefill_once(0)
        out["prefill"] = {k: v["share"] for k, v in kt.report().items()}
        ids = [f"k{i}" for i in range(B)]
        for r in ids:
            mgr.admit(r)
            mgr.grow(r, CTX - 8)
            mgr.commit(r, CTX - 8)
        step = lambda: llm.sampler.sample(runner.step([StepEntry(r, [1], [0]) for r in ids]), [(SamplingParams(), 0, 0)] * B)
        step()
        with KernelTimes() as kt:
            step()
        out["decode"] = {k: v["share"] for k, v in kt.report().items()}
        for r in ids:
            runner.finish(r)
        return out

    pre_clocks = ClockSampler()
    if args.section == "decode":
        pre_ms = own_ms = float("nan")
    else:
        for i in range(3):
            prefill_once(i)
        runner.check_status()
        pre_clocks.start()
        pre_ms = statistics.median(timed(prefill_once, 1) for _ in range(5))
        # for comparison: the same step with the library product (cuBLAS) in place of this package's tcgen05 kernel
        from llm_steadyinfer_b200.parts import linear as linear_mod
        was = linear_mod.USE_OWN_GEMM
        linear_mod.USE_OWN_GEMM = False
        for i in range(2):
            prefill_once(i)
        runner.check_status()
        own_ms = statistics.median(timed(prefill_once, 1) for _ in range(5))
        linear_mod.USE_OWN_GEMM = was
        pre_clocks.stop()
    if args.section == "prefill":
        print(json.dumps({"section": "prefill", "tokens": PT, "ms": round(pre_ms, 3), "library_gemm_ms": round(own_ms, 3)}))
        return 0
    pre_flops = 2 * PT * block_params + L * 4 * H * hs * PT * (PT + 1) / 2 + 2 * V * d
    prefill = {"value": round(PT / pre_ms * 1e3, 1), "tokens": PT, "ms": round(pre_ms, 3),
               "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "library_gemm_ms": round(own_ms, 3)}      # the same step with cuBLAS for the products (SI_OWN_GEMM=0)
    if "bf16_tflops_sustained" in pk:                     # the prompt step is tens of milliseconds of products
        prefill["frac_of_sustained"] = round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
    prefill["clocks"] = pre_clocks.summary()

    # ---- decode on the device: contexts filled synthetically, fixed next tokens ----------------
    for t in runner.storage.keys + runner.storage.values:
        t.normal_(0.0, 0.5)

    def decode_run(batch, steps, warm, sample=True, ctx_end=None):
        """``steps`` timed decode steps of ``batch`` requests after ``warm`` untimed ones; the contexts end at
        ``ctx_end`` tokens (default: the bench's context length)."""
        start = (ctx_end or CTX) - (steps + warm) - 1
        ids = [f"d{i}" for i in range(batch)]
        for r in ids:
            mgr.admit(r)
            mgr.grow(r, start)
            mgr.commit(r, start)
        toks = [rand_tokens(batch) for _ in range(steps + warm)]
        rows = [(SamplingParams(), 0, 0)] * batch
        state = {"i": 0}

        def one(_):
            entries = [StepEntry(r, [toks[state["i"]][j]], [0]) for j, r in enumerate(ids)]
            logits = runner.step_decode_graph(entries)
            if sample:
                llm.sampler.sample(logits, rows)
            state["i"] += 1

        for i in range(warm):
            one(i)
        runner.check_status()
        before = ops.launch_count()
        ms = timed(one, steps)
        launches = ops.launch_count() - before
        runner.check_status()
        for r in ids:
            runner.finish(r)
        mean_ctx = start + warm + (steps - 1) / 2 + 1
        return ms, launches, mean_ctx

    def hbm_frac(batch, mean_ctx, step_ms):
        """Bytes a decode step has to read (every weight once, the cache of the live requests) over its time."""
        step_bytes = weight_bytes + batch * mean_ctx * kv_bytes_per_token + batch * d * 2
        achieved = step_bytes / (step_ms * 1e-3) / 1e9
        return achieved, achieved / pk["hbm_gbs"]

    clocks.start()
    ms, launches, mean_ctx = decode_run(B, K, W)
    clocks.stop()
    ms_per_step = ms / K
    value = B * K / ms * 1e3
    achieved, frac = hbm_frac(B, mean_ctx, ms_per_step)
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(frac, 4), "peaks": pk_src}

    if args.section == "decode":
        print(json.dumps({"section": "decode", "ms_per_step": round(ms_per_step, 4), "roofline": roofline,
                          "gpu_launches": launches}))
        return 0
    # Further points: batch 1 and 64 at the bench's context, and the workload of the baseline configuration
    # (1,024-token prompts, 256 generated tokens: contexts from 1,024 to 1,280) at batch 1, 8 and 64. Each with
    # tokens a second, milliseconds a step and the fraction of the memory roofline.
    points = {}
    if not args.no_points:
        def point(name, b, steps, ctx_end=None):
            pm, _, mc = decode_run(b, steps, 4, ctx_end=ctx_end)
            points[name] = round(b * steps / pm * 1e3, 1)
            points[name + "_ms"] = round(pm / steps, 4)
            points[name + "_frac"] = round(hbm_frac(b, mc, pm / steps)[1], 4)
        for b in (1, 64):
            point(f"decode_b{b}", b, min(K, 32))
        for b in (1, 8, 64):
            point(f"decode_b{b}_ctx1280", b, 256, ctx_end=1280)
    kernel_times = {}
    if not args.no_points:
        kernel_times = kernel_time_shares()

    # ---- end to end through the Python entry point -------------------------------------------
    # The prompts are prefilled in portions, so the first requests decode while the last ones are still in
    # their prompts: every request gets room for those extra tokens, so that none ends inside the timed steps.
    ahead = B * (-(-CTX // 2048)) + 8
    plen = CTX - (K + W) - 2 - ahead
    for _ in range(B):
        llm.add_request(rand_tokens(plen), SamplingParams(max_tokens=K + W + 1 + ahead, ignore_eos=True))
    while any(not s.prefill_done for s in llm.get_running()) or llm.scheduler.waiting:
        llm.step()
    for _ in range(W):
        llm.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(K):
        llm.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if len(llm.get_running()) != B:
        raise RuntimeError("a request ended inside the timed end-to-end steps")
    e2e = {"value": round(B * K / e2e_s, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": runner.h2d_bytes_last_step,      # step inputs + attention work list
           "d2h_bytes_per_step": 4 * B + 4}                        # sampled ids + status word
    while not llm.all_finished():
        llm.step()

    out = {
        "metric": "decode tokens/s, Llama-3.1-8B shape, batch 8, context 8192", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights (seed 0), uniform random token ids", "impl": "ours",
        "config": {"model": "Llama-3.1-8B shape", "layers": L, "layers_full": layers_full, "hidden": d,
                   "heads": H, "kv_heads": KV, "head_dim": hs, "intermediate": F, "vocab": V,
                   "global_batch": B, "seq_len": CTX, "prefill_tokens": PT, "page_size": PAGE,
                   "parallelism": "single_gpu", "cuda_graph": True, "l2": "inputs larger than L2 (weights 16 GB)"},
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e, "kernel_time_shares": kernel_times,
        "gpu_launches": launches, "clocks": clocks.summary(),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
