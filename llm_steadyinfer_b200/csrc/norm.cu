// RMSNorm fused with the residual add that precedes it:
//   h = resid (+ delta);  resid <- h;  out = weight * h * rsqrt(mean(h^2) + eps)
// The reference runs the add (src/source/op/kernels/cuda/add_kernel.cu:4-12) and the
// norm (rmsnorm_kernel.cu:8-60, eps fixed at 1e-6) as separate launches; here eps is an
// argument, the residual stream is fp32, and sum of squares, mean and rsqrt are fp32.
// With `rows` given, output row r is computed from stream row rows[r] and the stream
// is left untouched (used to normalise only the rows whose logits are wanted).
#include "common.cuh"

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

template <typename TX>
static int launch(float* resid, const void* delta, const int* rows, const void* weight,
                  int weight_dtype, void* out, int num_rows, int hidden, float eps,
                  cudaStream_t stream) {
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return -2;           // hidden too large for the row cache
  if (weight_dtype == SI_BF16) {
    auto k = add_rmsnorm_kernel<TX, __nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<num_rows, threads, smem, stream>>>(resid, (const TX*)delta, rows,
                                           (const __nv_bfloat16*)weight, (TX*)out, hidden, eps);
  } else {
    auto k = add_rmsnorm_kernel<TX, float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<num_rows, threads, smem, stream>>>(resid, (const TX*)delta, rows, (const float*)weight,
                                           (TX*)out, hidden, eps);
  }
  return si_last_error();
}

// x_dtype: dtype of delta and out. Returns 0, a CUDA error code, or -2 (size refused).
SI_EXPORT int si_add_rmsnorm(float* resid, const void* delta, const int* rows, const void* weight,
                             int weight_dtype, void* out, int x_dtype, int num_rows, int hidden,
                             float eps, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (x_dtype == SI_BF16)
    return launch<__nv_bfloat16>(resid, delta, rows, weight, weight_dtype, out, num_rows, hidden, eps, stream);
  return launch<float>(resid, delta, rows, weight, weight_dtype, out, num_rows, hidden, eps, stream);
}
