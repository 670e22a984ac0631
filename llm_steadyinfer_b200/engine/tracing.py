"""Optional NVTX ranges around the phases of a step, for timelines of a profiler (nsys, ncu --nvtx): with
SI_NVTX=1 in the environment ``span(name)`` opens a range, otherwise it does nothing. The phases: "schedule",
"launch" and "resolve" in ``LLM.step``; "prepare", "forward" and "record" in the step function; "layer <i>" in
the model. The reference has no ranges; its drivers sample NVML and print VLOG lines per step
(benchmark/bench_common.h:110-161, src/source/scheduler/scheduler.cpp:140-164). Per-kernel device times are
``engine.kernel_times.KernelTimes``.
"""
from __future__ import annotations

import contextlib
import os

ENABLED = os.environ.get("SI_NVTX", "0") == "1"
_NOTHING = contextlib.nullcontext()


def span(name: str):
    """A context manager: an NVTX range named ``name`` when ranges are on, nothing otherwise."""
    if not ENABLED:
        return _NOTHING
    import torch
    return torch.cuda.nvtx.range(name)
