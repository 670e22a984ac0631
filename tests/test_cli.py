"""The command line: the reference's positional form and flags are parsed to the same fields."""
import json
import os
import subprocess
import sys

import pytest

from llm_steadyinfer_b200.cli.offline_batch_benchmark import parse_args

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_positional_form_and_flags():
    a = parse_args(["model_dir", "tok.json", "64", "16", "100", "out.csv", "2"])
    assert (a.checkpoint, a.tokenizer, a.num_requests, a.max_batch, a.max_gen, a.output_csv, a.iterations) == \
        ("model_dir", "tok.json", 64, 16, 100, "out.csv", 2)
    b = parse_args(["model_dir", "tok.json", "64", "16", "100", "--max-batch", "8", "--model-type", "llama3", "--seed", "7"])
    assert b.max_batch == 8 and b.num_requests == 64 and b.seed == 7
    c = parse_args(["--checkpoint", "m"])
    assert (c.num_requests, c.max_batch, c.max_gen, c.iterations, c.seed) == (512, 32, 256, 1, 42)    # the reference's defaults
    with pytest.raises(SystemExit):
        parse_args(["--checkpoint", "m", "--model-type", "qwen2"])
    with pytest.raises(SystemExit):
        parse_args([])


def test_gpu_sampler_against_a_stand_in_for_nvml():
    """The sampler thread averages what NVML returns and only reads; without NVML its figures stay 0."""
    import time
    import types
    from llm_steadyinfer_b200.cli.gpu_sampler import GpuUtilSampler, flops_per_token, peak_tflops
    calls = {"init": 0, "shutdown": 0, "reads": 0}

    def rates(dev):
        calls["reads"] += 1
        return types.SimpleNamespace(gpu=80 if calls["reads"] % 2 else 60, memory=30)

    fake = types.SimpleNamespace(
        nvmlInit=lambda: calls.__setitem__("init", calls["init"] + 1),
        nvmlShutdown=lambda: calls.__setitem__("shutdown", calls["shutdown"] + 1),
        nvmlDeviceGetHandleByIndex=lambda i: ("dev", i), nvmlDeviceGetUtilizationRates=rates,
        nvmlDeviceGetMemoryInfo=lambda dev: types.SimpleNamespace(used=3 * 1024 * 1024 * 1024))
    s = GpuUtilSampler(index=0, period_s=0.005, nvml=fake)
    assert s.start()
    time.sleep(0.08)
    s.stop()
    out = s.summary()
    assert out["gpu_samples"] >= 4 and 60 <= out["gpu_sm_util_pct"] <= 80 and out["gpu_mem_util_pct"] == 30
    assert out["gpu_mem_used_mb"] == 3072.0 and calls["init"] == 1 and calls["shutdown"] == 1
    broken = types.SimpleNamespace(nvmlInit=lambda: (_ for _ in ()).throw(RuntimeError("no driver")))
    b = GpuUtilSampler(nvml=broken)
    assert not b.start() and b.summary()["gpu_samples"] == 0
    b.stop()
    # the reference's estimate (benchmark/bench_common.h:215-221) at the Llama-3.1-8B sizes: 2 x the blocks' parameters
    assert flops_per_token(4096, 14336, 32, 32, 8, 128) == 32 * (4.0 * 4096 * 128 * 40 + 6.0 * 4096 * 14336)
    assert peak_tflops("bfloat16", 148, 1965.0, None) == (2250.0, "nominal dense bf16")
    v, src = peak_tflops("float32", 148, 1965.0, None)
    assert abs(v - 148 * 128 * 2 * 1.965e-3) < 1e-9 and "fp32" in src


@pytest.mark.gpu
def test_cli_runs_the_1b_style_workload_small(tmp_path):
    """Lognormal lengths, Poisson arrivals, a shared prefix, sampling: through the program itself."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from tiny_configs import make_model_folder
    folder = make_model_folder(tmp_path, "B")
    out = tmp_path / "m.json"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "offline_batch_benchmark"), "--checkpoint", folder,
         "--num-requests", "24", "--max-batch", "6", "--max-gen", "12", "--prompt-len-dist", "lognormal:40,0.8,4,150",
         "--output-len-dist", "lognormal:8,0.5,1,12", "--prefix-share", "0.4,32", "--request-rate", "400",
         "--temperature", "0.7", "--top-p", "0.9", "--ignore-eos", "--kv-block-size", "8", "--num-kv-blocks", "80",
         "--max-num-batched-tokens", "48", "--output-csv", str(tmp_path / "m.csv"), "--output-json", str(out)],
        capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    m = json.loads(out.read_text())[0]
    assert m["completed"] == 24 and m["rejected"] == 0 and m["output_tokens"] > 24
    assert m["prefix_hit_tokens"] > 0 and m["output_tps"] > 0 and m["ttft_p99_ms"] >= m["ttft_p50_ms"] > 0
    assert (tmp_path / "m.csv").read_text().startswith("run_id,")
    assert 0 < m["mfu"] < 1 and m["peak_tflops"] > 0
    # the reference's occupancy figures (offline_batch_benchmark.cpp:343-354)
    assert 0 < m["avg_decode_batch"] <= 6 and 0 < m["throughput_efficiency"] <= 1
    assert abs(m["throughput_efficiency"] - m["output_tps"] / m["theoretical_peak_tps"]) < 1e-3
    assert 0 < m["avg_busy_kv_slots"] <= m["peak_busy_kv_slots"] <= 6 and 0 <= m["kv_cache_frag_per_seq"] < 1
    assert m["avg_batch_reconstruct_ms"] > 0 and m["p99_batch_reconstruct_ms"] > 0     # (a recording can lift the mean above p99)
    assert {"gpu_sm_util_pct", "gpu_mem_util_pct", "gpu_mem_used_mb", "gpu_samples"} <= set(m)
