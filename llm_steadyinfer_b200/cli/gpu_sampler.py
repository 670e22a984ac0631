"""What the benchmark programs report about the GPU itself, in the manner of the reference's
``benchmark/bench_common.h``: utilisation and memory sampled through NVML every 50 ms by a thread of its own
(bench_common.h:110-161), and the model FLOPs utilisation from an estimate of the FLOPs per token
(bench_common.h:215-221). NVML is only read here (utilisation rates, memory in use); nothing is set.
"""
from __future__ import annotations

import json
import os
import threading
from typing import Optional


class GpuUtilSampler:
    """Mean SM utilisation, memory-controller utilisation and memory in use of one GPU while it runs.
    ``nvml``: a module with pynvml's functions (default: ``pynvml`` itself, if it can be imported; without it
    ``start`` returns False and every figure stays 0, as the reference's build without NVML)."""

    def __init__(self, index: int = 0, period_s: float = 0.05, nvml=None):
        self.index, self.period_s, self._nvml = index, period_s, nvml
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._dev = None
        self.samples = 0
        self._sm = self._mem = self._used_mb = 0.0

    def start(self) -> bool:
        if self._nvml is None:
            try:
                import pynvml
                self._nvml = pynvml
            except Exception:
                return False
        try:
            self._nvml.nvmlInit()
            self._dev = self._nvml.nvmlDeviceGetHandleByIndex(self.index)
        except Exception:
            return False
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return True

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                u = self._nvml.nvmlDeviceGetUtilizationRates(self._dev)
                self._sm += float(u.gpu)
                self._mem += float(u.memory)
                m = self._nvml.nvmlDeviceGetMemoryInfo(self._dev)
                self._used_mb += float(m.used) / (1024.0 * 1024.0)
                self.samples += 1
            except Exception:
                pass
            self._stop.wait(self.period_s)

    def stop(self) -> None:
        if self._thread is None:
            return
        self._stop.set()
        self._thread.join()
        self._thread = None
        try:
            self._nvml.nvmlShutdown()
        except Exception:
            pass

    def summary(self) -> dict:
        n = max(self.samples, 1)
        return {"gpu_sm_util_pct": round(self._sm / n, 2), "gpu_mem_util_pct": round(self._mem / n, 2),
                "gpu_mem_used_mb": round(self._used_mb / n, 1), "gpu_samples": self.samples}


def flops_per_token(hidden: int, intermediate: int, layers: int, heads: int, kv_heads: int, head_dim: int) -> float:
    """FLOPs of one token through the blocks' projections, the estimate behind the reference's MFU ("2 x
    parameters"; attention over the context left out, bench_common.h:215-221): q and o projections
    2 * 2 * d * H * hs, k and v 2 * 2 * d * KV * hs, gate, up and down 3 * 2 * d * F, a layer."""
    attn = 4.0 * hidden * head_dim * (heads + kv_heads)
    ffn = 6.0 * hidden * intermediate
    return layers * (attn + ffn)


def peak_tflops(dtype_name: str, sm_count: int, sm_clock_mhz: float, peaks_file: Optional[str] = None):
    """The rate MFU is taken against, and where it comes from. bfloat16: the measured cuBLAS rate in
    ``peaks_file`` (a JSON object with ``bf16_tflops``) when it is there, else the B200's nominal dense 2,250
    TFLOP/s. float32: the CUDA cores' 128 lanes x 2 x clock per SM, which is what the reference takes for every
    dtype (bench_common.h:166-192)."""
    if dtype_name == "bfloat16":
        if peaks_file and os.path.exists(peaks_file):
            try:
                with open(peaks_file) as f:
                    v = float(json.load(f)["bf16_tflops"])
                return v, "measured cuBLAS bf16"
            except Exception:
                pass
        return 2250.0, "nominal dense bf16"
    return sm_count * 128 * 2.0 * sm_clock_mhz / 1e6, "fp32 CUDA cores x clock"
