"""Python side of the CUDA kernels: thin wrappers that check shapes and dtypes, pass raw
device pointers and the current stream to the C entry points, and raise on any error.
Nothing here computes on the CPU or through a library: a missing build fails loudly.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


_c_int, _c_ll, _c_f, _c_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, found {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    """The tensor's address as ctypes takes it for a ``void*`` argument (an int, or None for a null pointer)."""
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_device_index: Optional[int] = None


def set_device(index: Optional[int]) -> None:
    """The device whose current stream the kernels are launched on, when the caller knows it (an engine that
    lives on one device); None: ask torch for the current device at every call."""
    global _device_index
    _device_index = index


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current one), asked once per device."""
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = _device_index if _device_index is not None else torch.cuda.current_device()
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return n


def _stream():
    """The current stream's handle. Every kernel call asks for it, so it comes from the one C call that
    returns the handle (torch.cuda.current_stream() builds a Python object around it at ten times the cost)."""
    if _raw_stream is not None:
        return _raw_stream(_device_index if _device_index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*ts) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors only; there is no CPU path")


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far in this process (graph replays are added by
    the code that replays them)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(rc: int, what: str, kernels: int = 1) -> None:
    global _launches
    if rc == 0:
        _launches += kernels
        return
    if rc == -2:
        raise KernelError(f"{what}: this size is outside what the kernel supports")
    raise KernelError(f"{what}: CUDA error {rc}")


_fn_cache = {}


def _fn(libname: str, symbol: str, argtypes):
    key = (libname, symbol)
    f = _fn_cache.get(key)
    if f is None:
        lib = build.load(libname)
        f = getattr(lib, symbol)
        f.argtypes = argtypes
        f.restype = _c_int
        _fn_cache[key] = f
    return f


def _i32(t: Optional[torch.Tensor], name: str) -> None:
    if t is not None:
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be contiguous int32")


# ---------------------------------------------------------------------------------------

def embedding_gather(tokens, table, out, status=None) -> None:
    """out[t,:] (fp32) = table[tokens[t],:]."""
    _cuda(tokens, table, out, status)
    _i32(tokens, "tokens")
    _need(out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous(),
          "embedding: out must be contiguous fp32, table contiguous")
    T, d = out.shape
    _need(table.shape[1] == d and tokens.numel() == T, "embedding: shape mismatch")
    f = _fn("embedding", "si_embedding_gather",
            [_c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(tokens), _ptr(table), _dt(table), _ptr(out), T, d, table.shape[0],
             _ptr(status), _stream()), "embedding_gather")


# Most bytes that one launch fetches ahead into L2. Measured on the 8B shape: 4 to 8 MB, what arrives while
# the norm waits on its own loads, shortened a decode step by 0.5 to 1.3 % while only the norms triggered the
# launch of the kernel after them; now that the products do too, 0 to 8 MB differ by less than half a per cent
# either way (4 MB is never the worst), and 16 MB and more still lengthen the step.
AHEAD_BYTES = int(os.environ.get("SI_AHEAD_MB", "4")) << 20


def add_rmsnorm(resid, delta, weight, eps: float, out, rows=None, ahead=None) -> None:
    """resid (fp32, in place) += delta; out = weight * resid * rsqrt(mean(resid^2) + eps).

    With ``rows`` (int32 [R]) output row r comes from stream row rows[r] and resid stays
    as it is. ``ahead``: a tensor that the kernel after this one streams from memory (weights of
    the next matrix product); further blocks of this launch start fetching it into L2.
    """
    _cuda(resid, delta, weight, out, rows)
    _i32(rows, "rows")
    d = resid.shape[-1]
    _need(resid.dtype == torch.float32 and resid.is_contiguous() and out.is_contiguous()
          and weight.is_contiguous(), "add_rmsnorm: tensors must be contiguous, resid fp32")
    _need(weight.numel() == d and out.shape[-1] == d, "add_rmsnorm: width mismatch")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == resid.shape,
              "add_rmsnorm: delta must match resid's shape and out's dtype")
    R = out.shape[0]
    _need(R == (rows.numel() if rows is not None else resid.shape[0]), "add_rmsnorm: row count mismatch")
    f = _fn("norm", "si_add_rmsnorm",
            [_c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_f, _c_p, _c_ll, _c_p])
    ahead_bytes = 0
    if ahead is not None:
        _cuda(ahead)
        ahead_bytes = min(ahead.numel() * ahead.element_size(), AHEAD_BYTES) if ahead.is_contiguous() else 0
    _check(f(_ptr(resid), _ptr(delta), _ptr(rows), _ptr(weight), _dt(weight), _ptr(out), _dt(out),
             R, d, float(eps), _ptr(ahead) if ahead_bytes else None, ahead_bytes, _stream()), f"add_rmsnorm(hidden={d})")


def rmsnorm_rows(x, weight, eps: float, out=None) -> None:
    """out[..., :] = weight * x[..., :] * rsqrt(mean(x[..., :]^2) + eps) over the last dimension of a 2-D or 3-D
    tensor (or view: only the last dimension must be contiguous), in place by default. No residual stream is
    involved: for norms inside a part (a norm over each head of a stacked projection, say)."""
    out = x if out is None else out
    _cuda(x, weight, out)
    _need(x.dim() in (2, 3) and out.shape == x.shape and out.dtype == x.dtype, "rmsnorm_rows: x and out must be 2-D or 3-D and alike")
    _need(x.stride(-1) == 1 and out.stride(-1) == 1 and weight.is_contiguous() and weight.numel() == x.shape[-1],
          "rmsnorm_rows: the last dimension must be contiguous and as long as the weight")
    if x.dim() == 2:
        rows, inner = x.shape[0], 1
        xs, os_ = (x.stride(0), 0), (out.stride(0), 0)
    else:
        rows, inner = x.shape[0] * x.shape[1], x.shape[1]
        xs, os_ = (x.stride(0), x.stride(1)), (out.stride(0), out.stride(1))
    f = _fn("norm", "si_rmsnorm_rows", [_c_p, _c_p, _c_int, _c_p, _c_int, _c_ll, _c_int, _c_int, _c_ll, _c_ll, _c_ll, _c_ll, _c_f, _c_p])
    _check(f(_ptr(x), _ptr(out), _dt(x), _ptr(weight), _dt(weight), rows, x.shape[-1], inner, xs[0], xs[1], os_[0], os_[1],
             float(eps), _stream()), f"rmsnorm_rows(n={x.shape[-1]})")


def rope_kv_write(qkv, positions, row_seq, inv_freq, rot_dim: int, block_table, k_cache, v_cache,
                  page_size: int, num_seqs: int, H: int, KV: int, hs: int, status=None) -> None:
    """Rotate q (in place) and k, store k and v of every row into its page.

    qkv: [T, (H+2KV)*hs]; k_cache/v_cache: [num_pages, KV, page_size, hs] of one layer, or None
    to rotate q only; inv_freq: fp32 [rot_dim/2] or None for no rotation.
    """
    _cuda(qkv, positions, row_seq, inv_freq, block_table, k_cache, v_cache, status)
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    T = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] == (H + 2 * KV) * hs, "rope_kv_write: qkv shape")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rot_dim,
              "rope_kv_write: inv_freq must be fp32 [rot_dim/2]")
    num_pages = 0
    if k_cache is not None:
        _need(k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype and k_cache.is_contiguous()
              and v_cache.is_contiguous(), "rope_kv_write: cache dtype/layout")
        _need(tuple(k_cache.shape[1:]) == (KV, page_size, hs) and k_cache.shape == v_cache.shape,
              "rope_kv_write: cache must be [pages, KV, page_size, hs]")
        num_pages = k_cache.shape[0]
    f = _fn("rope_kv", "si_rope_kv_write",
            [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(qkv), _dt(qkv), qkv.stride(0), _ptr(positions), _ptr(row_seq), _ptr(inv_freq),
             rot_dim, _ptr(block_table), block_table.shape[1], _ptr(k_cache), _ptr(v_cache),
             num_pages, page_size, T, num_seqs, H, KV, hs, _ptr(status), _stream()),
           f"rope_kv_write(head_dim={hs}, rot_dim={rot_dim})")


def paged_attention_ref(q, k_cache, v_cache, block_table, row_seq, positions, out, page_size: int,
                        num_seqs: int, H: int, KV: int, hs: int, scale: float, window: int = 0,
                        status=None) -> None:
    """Plain fp32-arithmetic attention over the paged cache; q may be a strided row view."""
    _cuda(q, k_cache, v_cache, block_table, row_seq, positions, out, status)
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    T = q.shape[0]
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == H * hs and out.shape[1] == H * hs,
          "paged_attention_ref: q/out shape")
    _need(q.dtype == out.dtype == k_cache.dtype == v_cache.dtype, "paged_attention_ref: dtypes differ")
    _need(tuple(k_cache.shape[1:]) == (KV, page_size, hs) and k_cache.is_contiguous()
          and v_cache.is_contiguous(), "paged_attention_ref: cache must be [pages, KV, page_size, hs]")
    f = _fn("attention_ref", "si_paged_attention_ref",
            [_c_p, _c_int, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p])
    _check(f(_ptr(q), _dt(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
             block_table.shape[1], _ptr(row_seq), _ptr(positions), _ptr(out), out.stride(0),
             k_cache.shape[0], page_size, T, num_seqs, H, KV, hs, float(scale), int(window or 0),
             _ptr(status), _stream()), f"paged_attention_ref(head_dim={hs})")


def swiglu(gu, out, group=None) -> None:
    """out[t,f] = silu(gate[t,f]) * up[t,f] from the stacked projection gu[t, 0..2F): gates and ups
    interleaved in groups of ``group`` columns (default F: all gates, then all ups)."""
    _cuda(gu, out)
    T, F = out.shape
    group = F if group is None else int(group)
    _need(gu.shape == (T, 2 * F) and gu.is_contiguous() and out.is_contiguous()
          and gu.dtype == out.dtype, "swiglu: gu must be [T, 2F] like out [T, F]")
    _need(group > 0 and F % group == 0, "swiglu: the group must divide F")
    f = _fn("swiglu", "si_swiglu", [_c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(gu), _ptr(out), _dt(out), T, F, group, _stream()), "swiglu")


def gemm_f32(a, w, out) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in true fp32 (FFMA)."""
    _cuda(a, w, out)
    _need(a.dtype == w.dtype == out.dtype == torch.float32, "gemm_f32: fp32 tensors only")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N) and a.stride(1) == 1 and w.stride(1) == 1
          and out.stride(1) == 1, "gemm_f32: shapes/strides")
    f = _fn("gemm_f32", "si_gemm_f32",
            [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K,
             _stream()), f"gemm_f32(M={M}, N={N}, K={K})")


def sample(logits, out, temperature=None, top_k=None, top_p=None, seed=None, counter=None) -> None:
    """Pick one token per row of fp32 logits; all per-row parameter tensors are optional
    (absent temperature means greedy)."""
    _cuda(logits, out, temperature, top_k, top_p, seed, counter)
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: logits must be fp32 rows")
    _i32(out, "out"); _i32(top_k, "top_k")
    R, V = logits.shape
    for t, dt, nm in ((temperature, torch.float32, "temperature"), (top_p, torch.float32, "top_p"),
                      (seed, torch.int64, "seed"), (counter, torch.int64, "counter")):
        if t is not None:
            _need(t.dtype == dt and t.numel() == R and t.is_contiguous(), f"sample: {nm} must be {dt} [rows]")
    f = _fn("sampling", "si_sample",
            [_c_p, _c_ll, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k), _ptr(top_p),
             _ptr(seed), _ptr(counter), _ptr(out), _stream()), "sample")


def argmax_scratch_words(rows: int) -> int:
    lib = build.load("sampling")
    lib.si_argmax_scratch_words.restype = _c_ll
    return int(lib.si_argmax_scratch_words(_c_int(rows)))


def argmax(logits, out, scratch) -> None:
    """Greedy pick per row of fp32 logits (ties to the lowest index) with the vocabulary of a row split over
    many blocks; ``scratch``: int32, ``argmax_scratch_words(capacity)`` long for some capacity >= rows,
    zeroed once by the caller and then left to this function."""
    _cuda(logits, out, scratch)
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "argmax: logits must be fp32 rows")
    _i32(out, "out"); _i32(scratch, "scratch")
    R, V = logits.shape
    capacity = scratch.numel() // argmax_scratch_words(1)
    _need(capacity >= R and scratch.is_contiguous(), "argmax: scratch too small")
    f = _fn("sampling", "si_argmax", [_c_p, _c_ll, _c_int, _c_int, _c_p, _c_int, _c_p, _c_p])
    _check(f(_ptr(logits), logits.stride(0), R, V, _ptr(scratch), capacity, _ptr(out), _stream()), "argmax")


def selftest_wait_runs_out(status, limit: int = 4096, gave_up=None) -> None:
    """Launch the self-test kernel whose bounded wait nothing ends: after ``limit`` probes it writes the
    wait-limit code into ``status`` (int32 [1]) and returns; ``gave_up`` (int32 [1], optional) is set to 1."""
    _cuda(status, gave_up)
    _i32(status, "status"); _i32(gave_up, "gave_up")
    f = _fn("selftest", "si_selftest_wait_runs_out", [_c_p, _c_int, _c_p, _c_p])
    _check(f(_ptr(status), int(limit), _ptr(gave_up), _stream()), f"selftest_wait_runs_out(limit={limit})")


# ---- tensor-core attention (bf16) ---------------------------------------------------------

_c_llr = ctypes.c_longlong


def attn_portion_tokens(H: int, KV: int, hs: int) -> int:
    """Most tokens of one item of the portion kernel (0: this head layout is not supported)."""
    lib = build.load("attention_mma")
    lib.si_attn_portion_tokens.restype = _c_int
    return lib.si_attn_portion_tokens(_c_int(H), _c_int(KV), _c_int(hs))


def attn_decode_rows(H: int, KV: int, hs: int) -> int:
    """Rows (tokens * heads per kv head) one item of the decode kernel may have; 0: none."""
    lib = build.load("attention_mma")
    lib.si_attn_decode_rows.restype = _c_int
    return lib.si_attn_decode_rows(_c_int(H), _c_int(KV), _c_int(hs))


def attn_decode_scratch_floats(num_items: int, H: int, KV: int, hs: int, nsplit: int) -> int:
    lib = build.load("attention_mma")
    lib.si_attn_decode_scratch_floats.restype = _c_llr
    return lib.si_attn_decode_scratch_floats(_c_int(num_items), _c_int(H), _c_int(KV), _c_int(hs), _c_int(nsplit))


def _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, what):
    _cuda(q, k_cache, v_cache, block_table, items, out)
    _i32(block_table, "block_table"); _i32(items, "items")
    _need(q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
          and v_cache.dtype == torch.bfloat16, f"{what}: bfloat16 tensors only")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == H * hs and out.shape[1] == H * hs,
          f"{what}: q/out must be [T, H*hs] rows")
    _need(tuple(k_cache.shape[1:]) == (KV, page_size, hs) and k_cache.is_contiguous() and v_cache.is_contiguous(),
          f"{what}: cache must be [pages, KV, page_size, hs]")
    _need(items.dim() == 2 and items.shape[1] == 4, f"{what}: items must be int32 [n, 4]")
    _need(q.data_ptr() % 16 == 0 and k_cache.data_ptr() % 16 == 0 and v_cache.data_ptr() % 16 == 0,
          f"{what}: q and cache must be 16-byte aligned")


def attn_portion(q, k_cache, v_cache, block_table, items, out, page_size: int, num_seqs: int, H: int,
                 KV: int, hs: int, scale: float, window: int = 0, status=None) -> None:
    """Tensor-core attention for prompt portions. ``items``: int32 [n, 4] rows
    (sequence, first row, tokens, first position), at most ``attn_portion_tokens`` tokens each."""
    _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, "attn_portion")
    f = _fn("attention_mma", "si_attn_portion",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_f, _c_int, _c_p, _c_p])
    _check(f(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
             _ptr(items), items.shape[0], _ptr(out), out.stride(0), k_cache.shape[0], page_size, num_seqs,
             H, KV, hs, float(scale), int(window or 0), _ptr(status), _stream()),
           f"attn_portion(heads={H}, kv_heads={KV}, head_dim={hs})")


def attn_decode(q, k_cache, v_cache, block_table, items, out, page_size: int, num_seqs: int, H: int, KV: int,
                hs: int, scale: float, window: int = 0, nsplit: int = 1, scratch=None, status=None) -> None:
    """Tensor-core attention for decode rows and short portions (at most
    ``attn_decode_rows // (H // KV)`` tokens an item). With ``nsplit`` > 1 the key range is split
    over blocks and ``scratch`` (fp32, ``attn_decode_scratch_floats`` elements, zero before its
    first use) holds the partials and the tickets of the merge."""
    _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, "attn_decode")
    if nsplit > 1:
        _cuda(scratch)
        need = attn_decode_scratch_floats(items.shape[0], H, KV, hs, nsplit)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need,
              f"attn_decode: scratch must hold {need} floats")
    f = _fn("attention_mma", "si_attn_decode",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_p, _c_p])
    _check(f(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
             _ptr(items), items.shape[0], _ptr(out), out.stride(0), k_cache.shape[0], page_size, num_seqs,
             H, KV, hs, float(scale), int(window or 0), int(nsplit), _ptr(scratch), _ptr(status), _stream()),
           f"attn_decode(heads={H}, kv_heads={KV}, head_dim={hs})")


# ---- decode attention with TMA-fed tiles ----------------------------------------------------

MAX_KEPT_MAPS = 4096      # descriptors kept per table; the oldest goes when a new one would exceed it


def _keep_map(table: dict, key, ent) -> None:
    """Descriptors are kept by (device, address, shape): a tensor at the same place with the same shape has
    the same descriptor, so an entry that outlives its tensor is still right for the next one there. The
    table is bounded, so that a process that builds engine after engine does not grow it for ever."""
    while len(table) >= MAX_KEPT_MAPS:
        table.pop(next(iter(table)))
    table[key] = ent


_tensor_maps = {}


def attn_decode_tma_ok(H: int, KV: int, hs: int, page_size: int) -> bool:
    """True when the TMA decode kernel takes this head layout and page size."""
    lib = build.load("attention_tma")
    lib.si_attn_decode_tma_ok.restype = _c_int
    return bool(lib.si_attn_decode_tma_ok(_c_int(H), _c_int(KV), _c_int(hs), _c_int(page_size)))


def attn_decode_tma_rows(H: int, KV: int) -> int:
    lib = build.load("attention_tma")
    lib.si_attn_decode_tma_rows.restype = _c_int
    return lib.si_attn_decode_tma_rows(_c_int(H), _c_int(KV))


def attn_decode_tma_scratch_floats(num_items: int, H: int, KV: int, hs: int, nsplit: int) -> int:
    lib = build.load("attention_tma")
    lib.si_attn_decode_tma_scratch_floats.restype = _c_llr
    return lib.si_attn_decode_tma_scratch_floats(_c_int(num_items), _c_int(H), _c_int(KV), _c_int(hs), _c_int(nsplit))


def _cache_map(cache: torch.Tensor):
    """The TMA descriptor of one layer's K or V cache; made once per tensor and kept."""
    key = (cache.device.index, cache.data_ptr(), tuple(cache.shape))
    ent = _tensor_maps.get(key)
    if ent is None:
        raw = ctypes.create_string_buffer(128 + 64)
        addr = (ctypes.addressof(raw) + 63) & ~63
        num_pages, KV, page_size, hs = cache.shape
        f = _fn("attention_tma", "si_attn_encode_cache_map", [_c_p, _c_p, _c_ll, _c_int, _c_int, _c_int])
        rc = f(_c_p(addr), _ptr(cache), num_pages, KV, page_size, hs)
        if rc != 0:
            raise KernelError(f"cannot describe the cache {tuple(cache.shape)} to the TMA unit (code {rc})")
        ent = (raw, addr)
        _keep_map(_tensor_maps, key, ent)
    return _c_p(ent[1])


def split_work(tiles, budget: int, entries: int, max_splits: int = 128, min_tiles: int = 1):
    """Cut decode items into shares of about equal length. ``tiles[i]``: 64-key tiles that item i reads
    (0: an empty item, which gets no entry). ``budget``: shares that run at the same time. With no more
    items than that, the shares are as short as ``budget`` shares in all allow (the smallest length L with
    sum(ceil(tiles / L)) <= budget): more would run in a second round, fewer would leave the longest item
    to few blocks. With more items than that the cut is chosen by an estimate of the time (see the code), so
    that a long item among many short ones is still cut and the last blocks do not run alone. No share is shorter than ``min_tiles``, no item has more than ``max_splits``. Returns
    an int32 array [entries, 4] of (item, split, splits of the item, first slot of the item), longest
    shares first, the rest filled with item -1: ``attn_decode_tma(work=...)``. ``entries >= budget +
    len(tiles)`` always suffices; more entries allow finer cuts when items outnumber the budget."""
    import numpy as np
    key = (tuple(tiles), budget, entries, max_splits, min_tiles)
    if _split_memo.get("key") == key:               # tile counts change once in 64 decode steps of a sequence
        return _split_memo["work"]
    _split_memo["key"], _split_memo["work"] = key, _split_work(np, tiles, budget, entries, max_splits, min_tiles)
    return _split_memo["work"]


_split_memo: dict = {}


def _split_work(np, tiles, budget, entries, max_splits, min_tiles):
    t = np.asarray(tiles, dtype=np.int64)
    live = np.flatnonzero(t > 0)
    out = np.full((entries, 4), -1, dtype=np.int32)
    out[:, 1:] = 0
    if live.size == 0:
        return out
    tl = t[live]

    def splits_for(L):
        return np.minimum(max_splits, -(-tl // max(L, min_tiles, 1)))

    if live.size <= budget:
        lo, hi = 1, int(tl.max())                    # smallest L whose shares fit the budget
        while lo < hi:
            mid = (lo + hi) // 2
            if int(splits_for(mid).sum()) <= budget:
                hi = mid
            else:
                lo = mid + 1
        sp = splits_for(lo)
    else:
        # More items than shares that run at once. Blocks follow one another on the block slots; what counts is
        # the longest chain on a slot (about ceil(shares / slots) shares of length L, at most load / slots + L),
        # the time HBM needs for everything (reached with about four fifths of the slots busy), and what a
        # share costs beside its tiles (about eight tiles' time for a full round of them: start, partial
        # results, merge). The cut with the least of these wins among 1 to 32 cuts of the longest item, as far
        # as the entries reach: many equal sequences stay whole, a few more sequences than slots are cut in
        # four or five so that the last blocks do not run alone, a long one among many short ones is cut most.
        load, slots, tmax = float(tl.sum()), float(max(budget, 1)), int(tl.max())
        best = None
        for k in (1, 2, 3, 4, 5, 6, 8, 12, 16, 32):
            L = max(-(-tmax // k), min_tiles, 1)
            cand = splits_for(L)
            n = int(cand.sum())
            if n > entries and best is not None:
                break
            longest = int((-(-tl // cand)).max())
            chain = min(-(-n // int(slots)) * longest, load / slots + longest)
            cost = max(chain, load / (0.8 * slots)) + 8.0 * n / slots
            if best is None or cost < best[0]:
                best = (cost, cand)
            if L <= max(min_tiles, 1):
                break
        sp = best[1]
    if int(sp.sum()) > entries:
        raise ValueError(f"split_work: {int(sp.sum())} shares do not fit {entries} entries")
    first = np.cumsum(sp) - sp
    order = np.argsort(-(-(-tl // sp)), kind="stable")          # longest shares first: they start first
    so = sp[order]
    total = int(so.sum())
    out[:total, 0] = np.repeat(live[order], so)
    out[:total, 1] = np.arange(total) - np.repeat(np.cumsum(so) - so, so)
    out[:total, 2] = np.repeat(so, so)
    out[:total, 3] = np.repeat(first[order], so)
    return out


_work_floats_memo: dict = {}


def attn_decode_tma_work_floats(slots: int, H: int, KV: int, hs: int) -> int:
    key = (slots, H, KV, hs)
    n = _work_floats_memo.get(key)
    if n is None:
        lib = build.load("attention_tma")
        lib.si_attn_decode_tma_work_floats.restype = _c_llr
        n = _work_floats_memo[key] = lib.si_attn_decode_tma_work_floats(_c_int(slots), _c_int(H), _c_int(KV), _c_int(hs))
    return n


def attn_decode_tma(q, k_cache, v_cache, block_table, items, out, page_size: int, num_seqs: int, H: int, KV: int,
                    hs: int, scale: float, window: int = 0, nsplit: int = 1, scratch=None, status=None,
                    max_rows: int = 0, work=None) -> None:
    """``attn_decode`` with the K/V tiles fetched by TMA (head_dim 64 or 128, page sizes 8 to 64);
    items hold at most ``attn_decode_tma_rows // (H // KV)`` tokens. ``max_rows``: the most rows
    (tokens x query heads of a KV head) of any item when the caller knows it (0: unknown); at most 8
    rows run the variant with the products taken the other way round.
    ``work`` (int32 [W, 4], rows of (item, split, splits of that item, first slot of that item); item -1:
    nothing): every item is cut into its own number of shares, ``nsplit`` is not used, and ``scratch``
    holds ``attn_decode_tma_work_floats(W, ...)`` floats. Made by ``split_work``."""
    _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, "attn_decode_tma")
    if work is not None:
        _cuda(work, scratch)
        _need(work.dtype == torch.int32 and work.dim() == 2 and work.shape[1] == 4 and work.is_contiguous(),
              "attn_decode_tma: work must be int32 [W, 4]")
        need = attn_decode_tma_work_floats(work.shape[0], H, KV, hs)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need,
              f"attn_decode_tma: scratch must hold {need} floats")
    elif nsplit > 1:
        _cuda(scratch)
        need = attn_decode_tma_scratch_floats(items.shape[0], H, KV, hs, nsplit)
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need,
              f"attn_decode_tma: scratch must hold {need} floats")
    f = _fn("attention_tma", "si_attn_decode_tma",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_p, _c_int, _c_int, _c_p, _c_int, _c_p, _c_p])
    W = work.shape[0] if work is not None else 0
    _check(f(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _cache_map(k_cache), _cache_map(v_cache),
             _ptr(block_table), block_table.shape[1], _ptr(items), items.shape[0], _ptr(out), out.stride(0),
             k_cache.shape[0], page_size, num_seqs, H, KV, hs, float(scale), int(window or 0), int(nsplit),
             _ptr(work), W, W, _ptr(scratch), int(max_rows), _ptr(status), _stream()),
           f"attn_decode_tma(heads={H}, kv_heads={KV}, head_dim={hs}, page_size={page_size})")


# ---- few-row matrix product (decode) ----------------------------------------------------------

SKINNY_MAX_ROWS = 16


def gemm_skinny_ok(a, w, out) -> bool:
    """True when the few-row kernel takes these tensors (bf16, at most 16 rows, K a multiple of 8)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
            and a.shape[0] <= SKINNY_MAX_ROWS and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and out.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(a, w, out, checked: bool = False) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T for M <= 16: the weights stream through mma.sync fragments.
    ``checked``: the caller has just asked ``gemm_skinny_ok`` for these tensors."""
    _cuda(a, w, out)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm_skinny: shapes")
    _need(checked or gemm_skinny_ok(a, w, out),
          "gemm_skinny: bf16 inputs, at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_skinny", "si_gemm_skinny",
            [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), _dt(out), M, N, K, _stream()),
           f"gemm_skinny(M={M}, N={N}, K={K})")


def gemm_skinny_swiglu(a, w, out, checked: bool = False) -> None:
    """out[M,F] = silu(gate) * up of a[M,K] @ w[2F,K]^T for M <= 16, the rows of w interleaved in groups of 8
    (8 gates, their 8 ups, ...): the activation runs in the product's epilogue."""
    _cuda(a, w, out)
    M, K = a.shape
    F = out.shape[1]
    _need(w.shape == (2 * F, K) and out.shape[0] == M and F % 8 == 0 and out.dtype == torch.bfloat16,
          "gemm_skinny_swiglu: w must be [2F, K], out [M, F] bf16, F a multiple of 8")
    _need(checked or gemm_skinny_ok(a, w, out), "gemm_skinny_swiglu: bf16 inputs, at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_skinny", "si_gemm_skinny_swiglu", [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, F, K, _stream()),
           f"gemm_skinny_swiglu(M={M}, F={F}, K={K})")


def gemm_skinny_qkv_rope(a, w, out, positions, row_seq, inv_freq, block_table, k_cache, v_cache, page_size: int,
                         num_seqs: int, H: int, KV: int, hs: int, status=None) -> None:
    """The stacked q/k/v projection of at most 16 rows with what ``rope_kv_write`` would do next in its epilogue:
    q and k heads rotated by their row's position (the whole head, rotate-half pairs), q written to
    ``out[:, :H*hs]``, k and v stored into the rows' cache pages (``k_cache`` None: nothing stored). The k and v
    columns of ``out`` are left as they are."""
    _cuda(a, w, out, positions, row_seq, inv_freq, block_table, k_cache, v_cache, status)
    _i32(positions, "positions"); _i32(row_seq, "row_seq"); _i32(block_table, "block_table")
    M, K = a.shape
    _need(w.shape == ((H + 2 * KV) * hs, K) and out.shape[0] == M and out.shape[1] >= H * hs and out.dtype == torch.bfloat16,
          "gemm_skinny_qkv_rope: w must be [(H + 2 KV) * hs, K], out [M, >= H * hs] bf16")
    _need(gemm_skinny_ok(a, w, out) and hs % 16 == 0, "gemm_skinny_qkv_rope: bf16 inputs, at most 16 rows, K a multiple of 8, "
          "16-byte aligned rows, head_dim a multiple of 16")
    _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == hs,
          "gemm_skinny_qkv_rope: inv_freq must be fp32 [head_dim / 2] (the whole head is rotated)")
    _need(positions.numel() == M and row_seq.numel() == M, "gemm_skinny_qkv_rope: one position and sequence per row")
    num_pages = 0
    if k_cache is not None:
        _need(k_cache.dtype == torch.bfloat16 and v_cache.dtype == torch.bfloat16 and k_cache.is_contiguous()
              and v_cache.is_contiguous() and tuple(k_cache.shape[1:]) == (KV, page_size, hs)
              and k_cache.shape == v_cache.shape, "gemm_skinny_qkv_rope: cache must be bf16 [pages, KV, page_size, hs]")
        num_pages = k_cache.shape[0]
    f = _fn("gemm_skinny", "si_gemm_skinny_qkv_rope",
            [_c_p, _c_ll, _c_p, _c_ll, _c_p, _c_ll, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_p,
             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, K, _ptr(positions), _ptr(row_seq),
             _ptr(inv_freq), _ptr(block_table), block_table.shape[1] if block_table is not None else 0, _ptr(k_cache),
             _ptr(v_cache), num_pages, page_size, num_seqs, H, KV, hs, _ptr(status), _stream()),
           f"gemm_skinny_qkv_rope(M={M}, heads={H}, kv_heads={KV}, head_dim={hs})")


# ---- tcgen05 matrix product (many rows) -------------------------------------------------------

_weight_maps = {}


_tc05_available = None


def gemm_tc05_available() -> bool:
    """True when the driver hands out the tensor-map encoder that the TMA-fed kernels need."""
    global _tc05_available
    if _tc05_available is None:
        lib = build.load("gemm_tc05")
        lib.si_gemm_tc05_ok.restype = _c_int
        _tc05_available = bool(lib.si_gemm_tc05_ok())
    return _tc05_available


def gemm_tc05_ok(a, w, out) -> bool:
    """True when the tcgen05 kernel takes these tensors (bf16, K a multiple of 8, aligned rows)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
            and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _weight_map(w: torch.Tensor, box_rows: int = 256):
    """The weight's TMA descriptor with boxes of ``box_rows`` rows (256: one CTA a tile; 128: a pair of CTAs)."""
    key = (w.device.index, w.data_ptr(), tuple(w.shape), w.stride(0), box_rows)
    ent = _weight_maps.get(key)
    if ent is None:
        raw = ctypes.create_string_buffer(128 + 64)
        addr = (ctypes.addressof(raw) + 63) & ~63
        f = _fn("gemm_tc05", "si_gemm_tc05_encode_weight", [_c_p, _c_p, _c_int, _c_int, _c_ll, _c_int])
        rc = f(_c_p(addr), _ptr(w), w.shape[0], w.shape[1], w.stride(0), box_rows)
        if rc != 0:
            raise KernelError(f"cannot describe the weight {tuple(w.shape)} to the TMA unit (code {rc})")
        ent = (raw, addr)
        _keep_map(_weight_maps, key, ent)
    return _c_p(ent[1])


def gemm_tc05(a, w, out, status=None) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory)."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm_tc05: shapes")
    _need(gemm_tc05_ok(a, w, out), "gemm_tc05: bf16 inputs, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_tc05", "si_gemm_tc05",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    half = _weight_map(w, 128) if M > 128 else None          # more than one tile of rows: pairs of CTAs take tiles together
    _check(f(_ptr(a), a.stride(0), _weight_map(w), half, _ptr(out), out.stride(0), _dt(out), M, N, K, _ptr(status),
             _stream()), f"gemm_tc05(M={M}, N={N}, K={K})")


def gemm_tc05_add(a, w, resid, status=None) -> None:
    """resid[M,N] (fp32) += a[M,K] @ w[N,K]^T on the tcgen05 tensor cores, each sum rounded to bf16 before the add
    (what storing the product in bf16 and adding it in the norm kernel gives)."""
    _cuda(a, w, resid, status)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and resid.shape == (M, N) and resid.dtype == torch.float32 and resid.stride(1) == 1,
          "gemm_tc05_add: resid must be fp32 [M, N] rows")
    _need(gemm_tc05_ok(a, w, resid), "gemm_tc05_add: bf16 inputs, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_tc05", "si_gemm_tc05_add", [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p, _c_p])
    half = _weight_map(w, 128) if M > 128 else None
    _check(f(_ptr(a), a.stride(0), _weight_map(w), half, _ptr(resid), resid.stride(0), M, N, K, _ptr(status), _stream()),
           f"gemm_tc05_add(M={M}, N={N}, K={K})")


def gemm_tc05_swiglu(a, w, out, status=None) -> None:
    """out[M,F] = silu(gate) * up of a[M,K] @ w[2F,K]^T on the tcgen05 tensor cores, the rows of w interleaved
    in groups of 8 (8 gates, their 8 ups, ...): the activation runs in the product's epilogue."""
    _cuda(a, w, out, status)
    M, K = a.shape
    F = out.shape[1]
    _need(w.shape == (2 * F, K) and out.shape[0] == M and F % 8 == 0 and out.dtype == torch.bfloat16,
          "gemm_tc05_swiglu: w must be [2F, K], out [M, F] bf16, F a multiple of 8")
    _need(gemm_tc05_ok(a, w, out), "gemm_tc05_swiglu: bf16 inputs, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_tc05", "si_gemm_tc05_swiglu", [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p, _c_p])
    half = _weight_map(w, 128) if M > 128 else None
    _check(f(_ptr(a), a.stride(0), _weight_map(w), half, _ptr(out), out.stride(0), M, F, K, _ptr(status), _stream()),
           f"gemm_tc05_swiglu(M={M}, F={F}, K={K})")


# ---- tcgen05 matrix product for up to 128 rows ------------------------------------------------------

ROWS_MAX = 128


def gemm_rows_ok(a, w, out) -> bool:
    """True when the product for up to 128 rows takes these tensors (bf16, K a multiple of 8, aligned rows)."""
    return a.shape[0] <= ROWS_MAX and gemm_tc05_ok(a, w, out)


def gemm_rows(a, w, out, status=None) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T for M <= 128 on the tcgen05 tensor cores: a tile of 128 output columns a
    block, the k range of a tile cut over a cluster where the tiles alone do not fill the GPU (see gemm_rows.cu)."""
    _cuda(a, w, out, status)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm_rows: shapes")
    _need(gemm_rows_ok(a, w, out), "gemm_rows: bf16 inputs, at most 128 rows, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_rows", "si_gemm_rows", [_c_p, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(a), a.stride(0), _weight_map(w, 128), _ptr(out), out.stride(0), _dt(out), M, N, K,
             _ptr(status), _stream()), f"gemm_rows(M={M}, N={N}, K={K})")


def gemm_rows_swiglu(a, w, out, status=None) -> None:
    """out[M,F] = silu(gate) * up of a[M,K] @ w[2F,K]^T for M <= 128, the rows of w interleaved in groups of 8
    (8 gates, their 8 ups, ...): the activation runs in the product's epilogue."""
    _cuda(a, w, out, status)
    M, K = a.shape
    F = out.shape[1]
    _need(w.shape == (2 * F, K) and out.shape[0] == M and F % 8 == 0 and out.dtype == torch.bfloat16,
          "gemm_rows_swiglu: w must be [2F, K], out [M, F] bf16, F a multiple of 8")
    _need(gemm_rows_ok(a, w, out), "gemm_rows_swiglu: bf16 inputs, at most 128 rows, K a multiple of 8, 16-byte aligned rows")
    f = _fn("gemm_rows", "si_gemm_rows_swiglu", [_c_p, _c_ll, _c_p, _c_p, _c_ll, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_ptr(a), a.stride(0), _weight_map(w, 128), _ptr(out), out.stride(0), M, F, K,
             _ptr(status), _stream()), f"gemm_rows_swiglu(M={M}, F={F}, K={K})")


# ---- prompt-portion attention on tcgen05 ---------------------------------------------------------

def attn_portion_tc05_ok(H: int, KV: int, hs: int, page_size: int) -> bool:
    lib = build.load("attention_tc05")
    lib.si_attn_portion_tc05_ok.restype = _c_int
    return bool(lib.si_attn_portion_tc05_ok(_c_int(H), _c_int(KV), _c_int(hs), _c_int(page_size)))


def attn_portion_tc05_tokens(H: int, KV: int) -> int:
    """Most tokens of one work item of ``attn_portion_tc05``."""
    lib = build.load("attention_tc05")
    lib.si_attn_portion_tc05_tokens.restype = _c_int
    return lib.si_attn_portion_tc05_tokens(_c_int(H), _c_int(KV))


def attn_portion_tc05(q, k_cache, v_cache, block_table, items, out, page_size: int, num_seqs: int, H: int,
                      KV: int, hs: int, scale: float, window: int = 0, status=None) -> None:
    """``attn_portion`` on the tcgen05 tensor cores (TMA-fed K/V tiles, S and P V in tensor memory);
    head_dim 64 or 128, page sizes 8 to 64, items of at most ``attn_portion_tc05_tokens`` tokens."""
    _attn_common(q, k_cache, v_cache, block_table, items, out, page_size, H, KV, hs, "attn_portion_tc05")
    f = _fn("attention_tc05", "si_attn_portion_tc05",
            [_c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_p, _c_ll, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p])
    _check(f(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _cache_map(k_cache), _cache_map(v_cache),
             _ptr(block_table), block_table.shape[1], _ptr(items), items.shape[0], _ptr(out), out.stride(0),
             k_cache.shape[0], page_size, num_seqs, H, KV, hs, float(scale), int(window or 0), _ptr(status),
             _stream()), f"attn_portion_tc05(heads={H}, kv_heads={KV}, head_dim={hs}, page_size={page_size})")
