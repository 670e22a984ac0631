"""Matrix products of the parts: ``out[M, N] = x[M, K] @ w[N, K]^T``.

fp32 tensors go through this package's own FFMA kernel (true 32-bit, no reduced-precision
mode). bf16 products of at most 16 rows (decode) go through the package's weight-streaming
kernel (``gemm_skinny.cu``). Other bf16 products go to the cuBLAS GEMM behind ``torch.mm`` with
fp32 accumulation, as the reference sends every projection and the LM head to ``cublasGemmEx``
(src/source/op/kernels/cuda/matmul_kernel.cu:128-150).
"""
from __future__ import annotations

import torch

from ..csrc import ops


USE_SKINNY = True      # few-row products (decode) through this package's weight-streaming kernel


def configure_library_gemm() -> None:
    """bf16 GEMMs accumulate in fp32 and are not allowed reduced-precision reductions."""
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_tf32 = False


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        raise ops.KernelError("linear: CUDA tensors only; there is no CPU path")
    if x.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32:
        ops.gemm_f32(x, w, out)
    elif USE_SKINNY and ops.gemm_skinny_ok(x, w, out):
        ops.gemm_skinny(x, w, out)
    elif x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if out.dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        elif out.dtype == torch.float32:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        else:
            raise ops.KernelError(f"linear: unsupported output dtype {out.dtype}")
    else:
        raise ops.KernelError(f"linear: unsupported dtypes x={x.dtype} w={w.dtype} out={out.dtype}")
    return out
