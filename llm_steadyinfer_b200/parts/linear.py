"""Matrix products of the parts: ``out[M, N] = x[M, K] @ w[N, K]^T``.

fp32 tensors go through this package's own FFMA kernel (true 32-bit, no reduced-precision
mode). bf16 products go by their number of rows: at most 16 (decode) to the package's
weight-streaming kernel on mma.sync (``gemm_skinny.cu``); 128 and more (prompt portions) to its
tcgen05 kernel, pairs of CTAs on 256 x 256 tiles (``gemm_tc05.cu``); 17 to 127 rows (larger decode
batches, short portions) to the library product behind ``torch.mm`` (cuBLAS, fp32 accumulation), as
the reference sends every projection and the LM head to ``cublasGemmEx``
(src/source/op/kernels/cuda/matmul_kernel.cu:128-150). The package has a tcgen05 kernel for those
row counts too (``gemm_rows.cu``, SI_OWN_ROWS=1 turns it on), but at the shapes measured the library
is still 1.1 to 1.6 times faster there. The library also takes what the kernels refuse (rows that are
not 16-byte aligned), and every many-row product with SI_OWN_GEMM=0.
"""
from __future__ import annotations

import os

import torch

from ..csrc import ops


USE_SKINNY = True      # few-row products (decode) through this package's weight-streaming kernel
USE_ROWS = os.environ.get("SI_OWN_ROWS", "0") == "1"      # 17 to 127 rows through gemm_rows.cu (default: the library)
USE_OWN_GEMM = os.environ.get("SI_OWN_GEMM", "1") == "1"  # 128 rows and more through gemm_tc05.cu (0: the library)
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


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status=None) -> torch.Tensor:
    """``status``: the engine's status word, where a kernel's bounded wait that ran out is reported."""
    if not x.is_cuda:
        raise ops.KernelError("linear: CUDA tensors only; there is no CPU path")
    if x.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype == torch.float32:
        ops.gemm_f32(x, w, out)
    elif USE_SKINNY and ops.gemm_skinny_ok(x, w, out):
        ops.gemm_skinny(x, w, out, checked=True)
    elif USE_ROWS and x.shape[0] < OWN_GEMM_MIN_ROWS and ops.gemm_tc05_available() and ops.gemm_rows_ok(x, w, out):
        ops.gemm_rows(x, w, out, status)
    elif (USE_OWN_GEMM and x.shape[0] >= OWN_GEMM_MIN_ROWS and ops.gemm_tc05_available()
          and ops.gemm_tc05_ok(x, w, out)):
        ops.gemm_tc05(x, w, out, status)
    elif x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        library_mm(x, w, out)
    else:
        raise ops.KernelError(f"linear: unsupported dtypes x={x.dtype} w={w.dtype} out={out.dtype}")
    return out


# Many-row products that end a mixer or a feed-forward can add into the residual stream themselves
# (gemm_tc05_add). Off: measured on the 8B shape the prompt step is 4 to 7 % slower with it, because the epilogue's
# strided fp32 read-modify-write no longer hides under the next tile's instructions.
FUSE_RESIDUAL = os.environ.get("SI_FUSE_RESIDUAL", "0") == "1"


def linear_into_residual(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, status=None) -> bool:
    """``resid += x @ w^T`` by the product's own epilogue, where a kernel of the package does that (bf16, at least
    ``OWN_GEMM_MIN_ROWS`` rows); False, and nothing done, where none does. The sums are rounded to bf16 before the
    add, as when ``linear`` stores them and the norm after it adds them."""
    if (FUSE_RESIDUAL and USE_OWN_GEMM and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and resid.dtype == torch.float32 and x.shape[0] >= OWN_GEMM_MIN_ROWS and ops.gemm_tc05_available()
            and ops.gemm_tc05_ok(x, w, resid)):
        ops.gemm_tc05_add(x, w, resid, status)
        return True
    return False
