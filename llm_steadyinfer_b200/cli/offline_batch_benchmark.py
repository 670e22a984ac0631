"""Offline batch benchmark: a set of requests through the engine, throughput and latency out.

In the manner of the reference's ``benchmark/offline_batch_benchmark.cpp``: the same positional
form ``<checkpoint> <tokenizer> <num_requests> <max_batch> <max_gen> [output_csv] [iterations]``
and the same flags (``--model-type --dataset --checkpoint --tokenizer --model-config --output-csv
--num-requests --max-batch --max-gen --iterations --seed``, offline_batch_benchmark.cpp:56-110),
the same protocol (model loaded once; two short warm-up requests through the same engine, left
out of the statistics, :218-231; occupancy of the cache sampled every step, :246-269) and the
same names of metrics (:146-181). The engine takes token ids, not text: ``--checkpoint`` is a
model folder (config.json + safetensors), ``--tokenizer`` is accepted and unused, and ``--dataset``
is a JSONL file of ``{"id": ..., "prompt_token_ids": [...]}``; without a dataset, prompts are
uniform random ids with lengths from ``--prompt-len`` or ``--prompt-len-dist``.
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import os
import random
import statistics
import sys
import time
from typing import List, Optional


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    argv = list(sys.argv[1:] if argv is None else argv)
    positional = []
    while argv and not argv[0].startswith("--"):
        positional.append(argv.pop(0))
    ap = argparse.ArgumentParser(prog="offline_batch_benchmark", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-type", default="llama", help="llama (alias llama3); the only architecture of this engine")
    ap.add_argument("--dataset", default=None, help="JSONL of {id, prompt_token_ids}; default: synthetic prompts")
    ap.add_argument("--checkpoint", default=None, help="model folder with config.json and safetensors")
    ap.add_argument("--tokenizer", default=None, help="accepted for compatibility; the engine takes token ids")
    ap.add_argument("--model-config", default=None, help="config.json for a random-weights model when no checkpoint is given")
    ap.add_argument("--output-csv", default="results/metrics.csv")
    ap.add_argument("--num-requests", type=int, default=512, help="0 = every sample of the dataset")
    ap.add_argument("--max-batch", type=int, default=32)
    ap.add_argument("--max-gen", type=int, default=256)
    ap.add_argument("--iterations", type=int, default=1)
    ap.add_argument("--seed", type=int, default=42)
    # what the reference takes from the environment or fixes in code
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-model-len", type=int, default=None, help="default: longest prompt + max-gen")
    ap.add_argument("--kv-block-size", type=int, default=None, help="default 8/16/32 by mean prompt length (scheduler.cpp:11-15)")
    ap.add_argument("--num-kv-blocks", type=int, default=None)
    ap.add_argument("--max-num-batched-tokens", default="adaptive", help="prompt tokens per step, or 'adaptive'")
    ap.add_argument("--admit-on-first-portion", action="store_true",
                    help="admit a request when the pages of its first portion are free (default: of its whole prompt)")
    ap.add_argument("--no-cuda-graph", action="store_true")
    ap.add_argument("--no-prefix-cache", action="store_true")
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--prompt-len-dist", default=None, help="lognormal:mean,sigma,min,max (mean in tokens)")
    ap.add_argument("--output-len-dist", default=None, help="lognormal:mean,sigma,min,max; default: --max-gen for all")
    ap.add_argument("--prefix-share", default=None, help="frac,len: this fraction of requests share one random prefix")
    ap.add_argument("--request-rate", type=float, default=float("inf"), help="Poisson arrivals per second; inf = all at once")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--output-json", default=None)
    args = ap.parse_args(argv)
    for name, val in zip(("checkpoint", "tokenizer", "num_requests", "max_batch", "max_gen", "output_csv", "iterations"),
                         positional):
        if getattr(args, name) == ap.get_default(name):         # an explicit flag wins over the position
            setattr(args, name, int(val) if name in ("num_requests", "max_batch", "max_gen", "iterations") else val)
    if args.model_type not in ("llama", "llama3"):
        ap.error(f"--model-type {args.model_type!r}: this engine holds the llama architecture only")
    if not args.checkpoint and not args.model_config:
        ap.error("give --checkpoint <model folder> or --model-config <config.json> (random weights)")
    return args


def _lognormal(spec: str, rng: random.Random) -> int:
    kind, rest = spec.split(":")
    if kind != "lognormal":
        raise ValueError(f"unknown distribution {kind!r}")
    mean, sigma, lo, hi = (float(x) for x in rest.split(","))
    return int(min(hi, max(lo, round(rng.lognormvariate(math.log(mean), sigma)))))


def load_prompts(args, vocab: int, rng: random.Random):
    prompts = []
    if args.dataset:
        with open(args.dataset, "r", encoding="utf-8") as f:
            for line in f:
                line = line.strip()
                if line:
                    prompts.append([int(t) for t in json.loads(line)["prompt_token_ids"]])
        rng.shuffle(prompts)
        if args.num_requests:
            prompts = prompts[:args.num_requests]
    else:
        share = None
        if args.prefix_share:
            frac, plen = args.prefix_share.split(",")
            share = (float(frac), [rng.randrange(vocab) for _ in range(int(plen))])
        for _ in range(args.num_requests or 512):
            n = _lognormal(args.prompt_len_dist, rng) if args.prompt_len_dist else args.prompt_len
            p = [rng.randrange(vocab) for _ in range(n)]
            if share and rng.random() < share[0]:
                p = share[1] + p
            prompts.append(p)
    out_lens = [(_lognormal(args.output_len_dist, rng) if args.output_len_dist else args.max_gen) for _ in prompts]
    return prompts, out_lens


def pct(xs, q):
    if not xs:
        return 0.0
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(math.ceil(q / 100.0 * len(xs))) - 1)]


def run_once(llm, prompts, out_lens, args, run_id: int, rng: random.Random) -> dict:
    from llm_steadyinfer_b200 import SamplingParams
    import torch
    sched = llm.scheduler
    # warm-up through the same engine, left out of the statistics
    warm = {llm.add_request([1, 2, 3], SamplingParams(max_tokens=4, ignore_eos=True)) for _ in range(2)}
    while not llm.all_finished():
        llm.step()
    torch.cuda.synchronize()
    llm.get_finished()
    arrivals = [0.0] * len(prompts)
    if math.isfinite(args.request_rate):
        t = 0.0
        for i in range(len(prompts)):
            t += rng.expovariate(args.request_rate)
            arrivals[i] = t
    mk = lambda i: SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                                  seed=args.seed * 100003 + i, max_tokens=out_lens[i], ignore_eos=args.ignore_eos)
    rejected, pending, ids = 0, list(range(len(prompts))), {}
    steps0, pre0, rec0 = sched.num_steps, sched.num_preemptions, sched.num_recomputed_tokens
    used_sum = alloc_sum = running_sum = samples = peak_pages = busy_sum = peak_busy = 0
    dec0 = llm.stats["steps_with_decode"]
    llm.decode_host_ms.clear()
    ps = llm.runner.page_size
    from .gpu_sampler import GpuUtilSampler
    gpu = GpuUtilSampler(torch.cuda.current_device())
    gpu.start()
    start = time.monotonic()
    while pending or not llm.all_finished():
        now = time.monotonic() - start
        while pending and arrivals[pending[0]] <= now:
            i = pending.pop(0)
            try:
                ids[llm.add_request(prompts[i], mk(i))] = i
            except ValueError:
                rejected += 1
        if llm.all_finished():
            time.sleep(min(0.001, max(0.0, arrivals[pending[0]] - now)))
            continue
        running = llm.get_running()
        if running:
            pages = sum(len(llm.runner.manager.table(0, s.id)) for s in running)
            used_sum += sum(s.num_computed for s in running)
            alloc_sum += pages * ps
            running_sum += len(running)
            peak_pages = max(peak_pages, pages)
            busy = len(llm.runner.manager.requests)          # requests that hold cache, preempted ones included
            busy_sum += busy
            peak_busy = max(peak_busy, busy)
            samples += 1
        llm.step()
    torch.cuda.synchronize()
    wall = time.monotonic() - start
    gpu.stop()
    fin = [s for s in llm.get_finished() if s.id not in warm and s.outputs]
    ttft = [(s.first_token_time - s.arrival_time) * 1e3 for s in fin]
    e2e = [(s.finish_time - s.arrival_time) * 1e3 for s in fin]
    tpot = [(e - t) / (len(s.outputs) - 1) for s, t, e in zip(fin, ttft, e2e) if len(s.outputs) > 1]
    itl = [(b - a) * 1e3 for s in fin for a, b in zip(s.token_times, s.token_times[1:])]
    prompt_tokens = sum(len(s.prompt) for s in fin)
    output_tokens = sum(len(s.outputs) for s in fin)
    mean = lambda xs: statistics.fmean(xs) if xs else 0.0
    # a request's own waste: the unused end of its last page (the reference, with one slot of max_seq_len per
    # request, counts the unused end of the slot: offline_batch_benchmark.cpp:301-302)
    per_seq_frag = [1.0 - n / (-(-n // ps) * ps) for n in (len(s.prompt) + len(s.outputs) for s in fin)]
    decode_steps = llm.stats["steps_with_decode"] - dec0
    host_ms = list(llm.decode_host_ms)
    # steps that drew at least one token (the reference counts its pure decode steps, and its first tokens come
    # from other steps: offline_batch_benchmark.cpp:343-354); as if each had drawn max_batch of them
    peak_tps = args.max_batch * decode_steps / wall if wall > 0 else 0.0
    return {
        "run_id": run_id, "num_requests": len(prompts), "completed": len(fin), "rejected": rejected,
        "prompt_tokens": prompt_tokens, "output_tokens": output_tokens, "total_tokens": prompt_tokens + output_tokens,
        "wall_time_s": round(wall, 4), "output_tps": round(output_tokens / wall, 2),
        "total_tps": round((prompt_tokens + output_tokens) / wall, 2), "qps": round(len(fin) / wall, 3),
        "ttft_avg_ms": round(mean(ttft), 3), "ttft_p50_ms": round(pct(ttft, 50), 3), "ttft_p99_ms": round(pct(ttft, 99), 3),
        "tpot_avg_ms": round(mean(tpot), 3), "tpot_p50_ms": round(pct(tpot, 50), 3), "tpot_p99_ms": round(pct(tpot, 99), 3),
        "itl_avg_ms": round(mean(itl), 3), "itl_p99_ms": round(pct(itl, 99), 3),
        "e2e_avg_ms": round(mean(e2e), 3), "e2e_p99_ms": round(pct(e2e, 99), 3),
        "kv_cache_util_global": round(used_sum / alloc_sum, 4) if alloc_sum else 0.0,
        "kv_cache_frag_global": round(1 - used_sum / alloc_sum, 4) if alloc_sum else 0.0,
        "kv_cache_frag_per_seq": round(mean(per_seq_frag), 4),
        "avg_busy_kv_slots": round(busy_sum / samples, 3) if samples else 0.0, "peak_busy_kv_slots": peak_busy,
        "avg_batch_reconstruct_ms": round(mean(host_ms), 4), "p99_batch_reconstruct_ms": round(pct(host_ms, 99), 4),
        "peak_kv_blocks": peak_pages, "avg_batch_size": round(running_sum / samples, 3) if samples else 0.0,
        "avg_decode_batch": round(output_tokens / decode_steps, 3) if decode_steps else 0.0,
        "throughput_efficiency": round(output_tokens / wall / peak_tps, 4) if peak_tps else 0.0,
        "theoretical_peak_tps": round(peak_tps, 2),
        "steps": sched.num_steps - steps0, "preemptions": sched.num_preemptions - pre0,
        "recomputed_tokens": sched.num_recomputed_tokens - rec0,
        "prefix_hit_tokens": sum(s.prefix_hit_tokens for s in fin),
        "finish_reasons": dict((r, sum(1 for s in fin if s.finish_reason == r)) for r in {s.finish_reason for s in fin}),
        **model_flops_utilisation(llm, (prompt_tokens + output_tokens) / wall), **gpu.summary(),
    }


def model_flops_utilisation(llm, total_tps: float) -> dict:
    """MFU as the reference reports it (offline_batch_benchmark.cpp:355-362): tokens a second times the FLOPs of
    a token's projections over a peak rate, here the peak of the dtype that computes."""
    import torch
    from .gpu_sampler import flops_per_token, peak_tflops
    cfg = llm.model.config
    dims = [getattr(cfg, k, None) for k in ("hidden_size", "intermediate_size", "num_hidden_layers",
                                            "num_attention_heads", "num_key_value_heads", "head_dim")]
    if any(d is None for d in dims):
        return {"mfu": 0.0, "peak_tflops": 0.0, "peak_source": "no estimate for this architecture"}
    per_token = flops_per_token(*dims)
    prop = torch.cuda.get_device_properties(torch.cuda.current_device())
    clock_mhz = getattr(prop, "clock_rate", 0) / 1e3 or 1965.0
    here = os.path.dirname(os.path.abspath(__file__))
    peak, source = peak_tflops("bfloat16" if llm.dtype == torch.bfloat16 else "float32", prop.multi_processor_count, clock_mhz,
                               os.path.join(here, "..", "..", "MEASURED_PEAKS.json"))
    return {"mfu": round(total_tps * per_token / (peak * 1e12), 6), "peak_tflops": round(peak, 1), "peak_source": source}


def main(argv: Optional[List[str]] = None) -> int:
    args = parse_args(argv)
    import torch
    from llm_steadyinfer_b200 import LLM
    from llm_steadyinfer_b200.models import Model
    from llm_steadyinfer_b200.weights import init_random, load_model

    rng = random.Random(args.seed)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    if args.checkpoint:
        model = load_model(args.checkpoint, dtype, "cuda:0")
    else:
        from llm_steadyinfer_b200.config import config_from_dict
        with open(args.model_config) as f:
            model = Model(config_from_dict(json.load(f)), dtype, "cuda:0")
        init_random(model, args.seed)
    vocab = model.spec.vocab_size
    prompts, out_lens = load_prompts(args, vocab, rng)
    longest = max(len(p) for p in prompts)
    max_len = args.max_model_len or min(longest + max(out_lens), model.spec.max_position or 1 << 30)
    mean_len = sum(len(p) for p in prompts) / len(prompts)
    block = args.kv_block_size or (8 if mean_len < 64 else (32 if mean_len > 1024 else 16))
    budget = args.max_num_batched_tokens if args.max_num_batched_tokens == "adaptive" else int(args.max_num_batched_tokens)
    llm = LLM(model, dtype=dtype, max_batch=args.max_batch, max_seq_len=max_len, max_gen_len=args.max_gen,
              block_size=block, num_blocks=args.num_kv_blocks, max_num_batched_tokens=budget,
              enable_prefix_cache=not args.no_prefix_cache, use_cuda_graph=not args.no_cuda_graph,
              reserve="portion" if args.admit_on_first_portion else "prompt")
    rows = []
    for it in range(args.iterations):
        m = run_once(llm, prompts, out_lens, args, it, rng)
        rows.append(m)
        print(f"[run {it}] requests {m['completed']}/{m['num_requests']}  output_tps {m['output_tps']}  total_tps {m['total_tps']}  "
              f"ttft p50/p99 {m['ttft_p50_ms']}/{m['ttft_p99_ms']} ms  tpot p50/p99 {m['tpot_p50_ms']}/{m['tpot_p99_ms']} ms  "
              f"avg batch {m['avg_batch_size']}  preemptions {m['preemptions']}  prefix hit tokens {m['prefix_hit_tokens']}  "
              f"mfu {m['mfu']}  gpu sm/mem util {m['gpu_sm_util_pct']}/{m['gpu_mem_util_pct']} %")
    if args.output_csv:
        os.makedirs(os.path.dirname(os.path.abspath(args.output_csv)), exist_ok=True)
        with open(args.output_csv, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=list(rows[0].keys()))
            wr.writeheader()
            for r in rows:
                wr.writerow(r)
    if args.output_json:
        with open(args.output_json, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
