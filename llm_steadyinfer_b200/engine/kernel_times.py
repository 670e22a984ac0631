"""Device time per kind of kernel, measured with CUDA events around every kernel call of a step.

    with KernelTimes() as kt:
        runner.step(entries)            # a direct step (a recorded graph has no calls to time)
    kt.report()  ->  {"gemm_skinny": {"calls": 129, "ms": 3.41, "share": 0.78}, ...}

While it is active every launching function of ``csrc.ops`` and the library product of ``parts.linear`` is
wrapped: an event before and one after the call on the current stream. The events sit between the kernels, so
a kernel cannot start under the tail of the one before it (programmatic dependent launch) and the step takes
longer than it does unobserved: read the shares, and take absolute times from an unobserved run. The
reference's drivers print model FLOPs utilisation and NVML samples (benchmark/bench_common.h:110-221); a
breakdown by kernel is this package's addition.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..csrc import ops
from ..parts import linear as linear_mod

# launching functions of csrc.ops -> the name they are reported under
KINDS = {
    "embedding_gather": "embedding", "add_rmsnorm": "add_rmsnorm", "rope_kv_write": "rope_kv_write",
    "paged_attention_ref": "attention_ref", "swiglu": "swiglu", "gemm_f32": "gemm_f32",
    "sample": "sampling", "argmax": "sampling", "attn_portion": "attn_portion_mma", "attn_decode": "attn_decode_mma",
    "attn_decode_tma": "attn_decode_tma", "attn_portion_tc05": "attn_portion_tc05", "gemm_skinny": "gemm_skinny",
    "gemm_skinny_swiglu": "gemm_skinny_swiglu", "gemm_skinny_qkv_rope": "gemm_skinny_qkv_rope", "gemm_tc05": "gemm_tc05", "gemm_tc05_swiglu": "gemm_tc05_swiglu",
    "gemm_rows": "gemm_rows", "gemm_rows_swiglu": "gemm_rows_swiglu",
}


class KernelTimes:
    def __init__(self):
        self._events: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        self._saved: List[Tuple[object, str, object]] = []

    def _wrap(self, owner, attr: str, kind: str) -> None:
        fn = getattr(owner, attr, None)
        if fn is None:
            return
        events = self._events

        def timed(*args, **kwargs):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                return fn(*args, **kwargs)
            finally:
                b.record()
                events.append((kind, a, b))

        self._saved.append((owner, attr, fn))
        setattr(owner, attr, timed)

    def __enter__(self) -> "KernelTimes":
        for attr, kind in KINDS.items():
            self._wrap(ops, attr, kind)
        self._wrap(linear_mod, "library_mm", "library_gemm")
        return self

    def __exit__(self, *exc) -> None:
        for owner, attr, fn in reversed(self._saved):
            setattr(owner, attr, fn)
        self._saved.clear()

    def report(self) -> Dict[str, Dict[str, float]]:
        """Per kind: calls, milliseconds and share of the summed kernel time (waits for the device)."""
        torch.cuda.synchronize()
        acc: Dict[str, List[float]] = {}
        for kind, a, b in self._events:
            ent = acc.setdefault(kind, [0, 0.0])
            ent[0] += 1
            ent[1] += a.elapsed_time(b)
        total = sum(v[1] for v in acc.values()) or 1.0
        return {k: {"calls": int(v[0]), "ms": round(v[1], 4), "share": round(v[1] / total, 4)}
                for k, v in sorted(acc.items(), key=lambda kv: -kv[1][1])}
