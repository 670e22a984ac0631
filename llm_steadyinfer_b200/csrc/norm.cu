// RMSNorm fused with the residual add that precedes it:
//   h = resid (+ delta);  resid <- h;  out = weight * h * rsqrt(mean(h^2) + eps)
// The reference runs the add (src/source/op/kernels/cuda/add_kernel.cu:4-12) and the
// norm (rmsnorm_kernel.cu:8-60, eps fixed at 1e-6) as separate launches; here eps is an
// argument, the residual stream is fp32, and sum of squares, mean and rsqrt are fp32.
// With `rows` given, output row r is computed from stream row rows[r] and the stream
// is left untouched (used to normalise only the rows whose logits are wanted).
//
// One block per row. When the width is a multiple of 8 every thread moves 8 elements at a
// time with 16-byte loads (all loads of a row are in flight before the first use) and keeps
// them in registers between the two passes; other widths take the scalar kernel, which
// stages the row in shared memory.
#include "common.cuh"

template <typename T> struct Vec8;
template <> struct Vec8<float> {
  float v[8];
  __device__ __forceinline__ void load(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  __device__ __forceinline__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Vec8<__nv_bfloat16> {
  float v[8];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

// CHUNKS: 8-element chunks per thread (hidden <= CHUNKS * 8 * blockDim.x)
template <typename TX, typename TW, int CHUNKS>
__global__ void __launch_bounds__(512) add_rmsnorm_vec_kernel(float* __restrict__ resid, const TX* __restrict__ delta,
                                       const int* __restrict__ rows, const TW* __restrict__ weight,
                                       TX* __restrict__ out, int hidden, float eps, int num_rows,
                                       const void* ahead, long long ahead_bytes, int trigger) {
  __shared__ float scratch[33];
  if (trigger) pdl_trigger();
  if ((int)blockIdx.x >= num_rows) {              // blocks behind the rows only fetch ahead
    l2_prefetch_share(ahead, ahead_bytes, blockIdx.x - num_rows, gridDim.x - num_rows);
    return;
  }
  pdl_prologue();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* h = resid + (size_t)src * hidden;
  const TX* dl = delta ? delta + (size_t)src * hidden : nullptr;
  const int nchunks = hidden >> 3;
  Vec8<float> x[CHUNKS];
  Vec8<TX> dv[CHUNKS];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      x[c].load(h + ch * 8);
      if (dl) dv[c].load(dl + ch * 8);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      if (dl) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[c].v[i] += dv[c].v[i];
        if (!rows) x[c].store(h + ch * 8);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[c].v[i] * x[c].v[i];
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TX* o = out + (size_t)r * hidden;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int ch = threadIdx.x + c * blockDim.x;
    if (ch < nchunks) {
      Vec8<TW> w;
      w.load(weight + ch * 8);
      Vec8<TX> y;
#pragma unroll
      for (int i = 0; i < 8; ++i) y.v[i] = w.v[i] * (x[c].v[i] * inv);
      y.store(o + ch * 8);
    }
  }
}

template <typename TX, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TX* __restrict__ delta,
                                   const int* __restrict__ rows, const TW* __restrict__ weight,
                                   TX* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];        // `hidden` floats
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* h = resid + (size_t)src * hidden;
  const TX* dl = delta ? delta + (size_t)src * hidden : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = h[i];
    if (dl) v += to_f32<TX>(dl[i]);
    row_cache[i] = v;
    if (dl && !rows) h[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  TX* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_f32<TX>(to_f32<TW>(weight[i]) * (row_cache[i] * inv));
}

template <typename TX, typename TW>
static int launch2(float* resid, const void* delta, const int* rows, const void* weight, void* out,
                   int num_rows, int hidden, float eps, const void* ahead, long long ahead_bytes, cudaStream_t stream) {
  const TX* d = (const TX*)delta;
  const TW* w = (const TW*)weight;
  TX* o = (TX*)out;
  const bool aligned = ((uintptr_t)resid % 16 == 0) && ((uintptr_t)delta % 16 == 0) &&
                       ((uintptr_t)weight % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (hidden % 8 == 0 && aligned && hidden <= 4 * 8 * 512) {
    const int nchunks = hidden / 8;
    // threads: a multiple of 32 that covers the row in at most 4 passes
    int threads = nchunks > 256 ? 512 : (nchunks > 128 ? 256 : 128);
    if (num_rows >= 1024 && nchunks <= 1024) threads = min(threads, 256);   // many rows: more blocks per SM
    const int per = (nchunks + threads - 1) / threads;
    // with something to fetch ahead: enough further blocks that every SM takes part
    if (ahead && ahead_bytes < 4096) ahead = nullptr;
    const int trigger = si_pdl_trigger_enabled() && num_rows <= 64;      // a launch of one wave
    const int sms = si_sm_count();
    const int extra = ahead ? max(0, sms - num_rows) + sms : 0;
    const dim3 grid(num_rows + extra);
    if (per <= 1) si_launch(add_rmsnorm_vec_kernel<TX, TW, 1>, grid, dim3(threads), 0, stream, resid, d, rows, w, o, hidden, eps, num_rows, ahead, ahead_bytes, trigger);
    else if (per <= 2) si_launch(add_rmsnorm_vec_kernel<TX, TW, 2>, grid, dim3(threads), 0, stream, resid, d, rows, w, o, hidden, eps, num_rows, ahead, ahead_bytes, trigger);
    else si_launch(add_rmsnorm_vec_kernel<TX, TW, 4>, grid, dim3(threads), 0, stream, resid, d, rows, w, o, hidden, eps, num_rows, ahead, ahead_bytes, trigger);
    return si_last_error();
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return -2;           // hidden too large for the row cache
  auto k = add_rmsnorm_kernel<TX, TW>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  k<<<num_rows, threads, smem, stream>>>(resid, d, rows, w, o, hidden, eps);
  return si_last_error();
}

// x_dtype: dtype of delta and out. `ahead` (may be null): `ahead_bytes` bytes that the kernel after this
// one streams, fetched into L2 meanwhile (a hint: the vectorised kernel takes it, the other one ignores it).
// Returns 0, a CUDA error code, or -2 (size refused).
SI_EXPORT int si_add_rmsnorm(float* resid, const void* delta, const int* rows, const void* weight,
                             int weight_dtype, void* out, int x_dtype, int num_rows, int hidden,
                             float eps, const void* ahead, long long ahead_bytes, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (x_dtype == SI_BF16) {
    if (weight_dtype == SI_BF16)
      return launch2<__nv_bfloat16, __nv_bfloat16>(resid, delta, rows, weight, out, num_rows, hidden, eps, ahead, ahead_bytes, stream);
    return launch2<__nv_bfloat16, float>(resid, delta, rows, weight, out, num_rows, hidden, eps, ahead, ahead_bytes, stream);
  }
  if (weight_dtype == SI_BF16)
    return launch2<float, __nv_bfloat16>(resid, delta, rows, weight, out, num_rows, hidden, eps, ahead, ahead_bytes, stream);
  return launch2<float, float>(resid, delta, rows, weight, out, num_rows, hidden, eps, ahead, ahead_bytes, stream);
}

// ---- a norm that is not on the residual stream ------------------------------------------------------------------
// out[r, :] = weight * x[r, :] * rsqrt(mean(x[r, :]^2) + eps) for rows of `n` elements that lie in a two-level
// layout: row r = (a, b) with b < inner starts at x + a * outer_stride + b * inner_stride (the heads of a token
// inside a stacked projection, for a norm over each head; inner = 1 for plain rows). One warp a row, statistics in
// fp32, in place if out == x. Nothing is added and no stream is written: what a mixer calls for a norm of its own.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const TX* __restrict__ x, TX* __restrict__ out,
                                                           const TW* __restrict__ weight, long long num_rows, int n, int inner,
                                                           long long x_outer, long long x_inner, long long o_outer,
                                                           long long o_inner, float eps) {
  pdl_prologue();
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= num_rows) return;
  const int lane = threadIdx.x & 31;
  const long long a = r / inner, b = r - a * inner;
  const TX* xr = x + a * x_outer + b * x_inner;
  TX* orow = out + a * o_outer + b * o_inner;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) {
    const float v = to_f32<TX>(xr[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)n + eps);
  for (int i = lane; i < n; i += 32) orow[i] = from_f32<TX>(to_f32<TW>(weight[i]) * (to_f32<TX>(xr[i]) * inv));
}

template <typename TX, typename TW>
static int rows_launch(const void* x, void* out, const void* weight, long long num_rows, int n, int inner, long long x_outer,
                       long long x_inner, long long o_outer, long long o_inner, float eps, cudaStream_t stream) {
  const long long blocks = (num_rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return -2;
  si_launch(rmsnorm_rows_kernel<TX, TW>, dim3((unsigned)blocks), dim3(256), 0, stream, (const TX*)x, (TX*)out, (const TW*)weight,
            num_rows, n, inner, x_outer, x_inner, o_outer, o_inner, eps);
  return si_last_error();
}

// x_dtype: dtype of x and out; strides in elements. Returns 0, a CUDA error code, or -2 (size refused).
SI_EXPORT int si_rmsnorm_rows(const void* x, void* out, int x_dtype, const void* weight, int weight_dtype, long long num_rows,
                              int n, int inner, long long x_outer, long long x_inner, long long o_outer, long long o_inner,
                              float eps, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (n <= 0 || inner <= 0) return -2;
  if (x_dtype == SI_BF16) {
    if (weight_dtype == SI_BF16)
      return rows_launch<__nv_bfloat16, __nv_bfloat16>(x, out, weight, num_rows, n, inner, x_outer, x_inner, o_outer, o_inner, eps, stream);
    return rows_launch<__nv_bfloat16, float>(x, out, weight, num_rows, n, inner, x_outer, x_inner, o_outer, o_inner, eps, stream);
  }
  if (weight_dtype == SI_BF16) return -2;
  return rows_launch<float, float>(x, out, weight, num_rows, n, inner, x_outer, x_inner, o_outer, o_inner, eps, stream);
}

