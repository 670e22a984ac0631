"""Matrix products of the parts: ``out[M, N] = x[M, K] @ w[N, K]^T``.

fp32 tensors go through this package's own FFMA kernel (true 32-bit, no reduced-precision
mode). bf16 products of at most 16 rows (decode) go through the package's weight-streaming
kernel (``gemm_skinny.cu``). Other bf16 products go to the cuBLAS GEMM behind ``torch.mm`` with
fp32 accumulation, as the reference sends every projection and the LM head to ``cublasGemmEx``
(src/source/op/kernels/cuda/matmul_kernel.cu:128-150), or, with ``USE_OWN_GEMM``, to the package's
tcgen05 kernel (``gemm_tc05.cu``).
"""
from __future__ import annotations

import os

import torch

from ..csrc import ops


USE_SKINNY = True      # few-row products (decode) through this package's weight-streaming kernel
# Many-row bf16 products (at least OWN_GEMM_MIN_ROWS rows) through this package's tcgen05 kernel instead of
# the library. Off by default: on the plain projections the library's 2-CTA kernels are 8 to 19 % faster
# (the gate/up projection, where the fused activation makes up for it, does not come through here).
# SI_OWN_GEMM=1 in the environment turns it on.
USE_OWN_GEMM = os.environ.get("SI_OWN_GEMM", "0") == "1"
OWN_GEMM_MIN_ROWS = 128


def configure_library_gemm() -> None:
    """bf16 GEMMs accumulate in fp32 and are not allowed reduced-precision reductions."""
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_tf32 = False


def library_mm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """The library product (cuBLAS behind ``torch.mm``), bf16 inputs, fp32 accumulation."""
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    elif out.dtype == torch.float32:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        raise ops.KernelError(f"linear: unsupported output dtype {out.dtype}")


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        raise ops.KernelError("linear: CUDA tensors only; there is no CPU path")
    if x.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32:
        ops.gemm_f32(x, w, out)
    elif USE_SKINNY and ops.gemm_skinny_ok(x, w, out):
        ops.gemm_skinny(x, w, out, checked=True)
    elif (USE_OWN_GEMM and x.shape[0] >= OWN_GEMM_MIN_ROWS and ops.gemm_tc05_available()
          and ops.gemm_tc05_ok(x, w, out)):
        ops.gemm_tc05(x, w, out)
    elif x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        library_mm(x, w, out)
    else:
        raise ops.KernelError(f"linear: unsupported dtypes x={x.dtype} w={w.dtype} out={out.dtype}")
    return out
