// Gated activation of the feed-forward: out[t, f] = silu(gu[t, f]) * gu[t, F + f], where
// gu is the output of the stacked gate/up projection. silu(x) = x / (1 + exp(-x)) in fp32,
// as the reference computes it (src/source/op/kernels/cuda/swiglu_kernel.cu:4-22).
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / F;
  const int f = (int)(idx - t * F);
  const T* row = gu + (size_t)t * 2 * F;
  const float g = to_f32<T>(row[f]);
  const float u = to_f32<T>(row[F + f]);
  out[idx] = from_f32<T>((g / (1.f + expf(-g))) * u);
}

SI_EXPORT int si_swiglu(const void* gu, void* out, int dtype, int num_tokens, int F,
                        cudaStream_t stream) {
  const long long total = (long long)num_tokens * F;
  if (total <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  if (dtype == SI_BF16)
    swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gu,
                                                                 (__nv_bfloat16*)out, F, total);
  else
    swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, F, total);
  return si_last_error();
}
