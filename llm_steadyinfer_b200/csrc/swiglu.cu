// Gated activation of the feed-forward: out[t, f] = silu(gate[t, f]) * up[t, f], where gate and up
// are the output gu[t, 0 .. 2F) of the stacked gate/up projection, interleaved in groups of `group`
// columns: gate f stands in column (f / group) * 2 * group + f % group and up f `group` columns
// further (group = F: all gates, then all ups). silu(x) = x / (1 + exp(-x)) in fp32,
// as the reference computes it (src/source/op/kernels/cuda/swiglu_kernel.cu:4-22).
// When the group is a multiple of 8 (4 for fp32) and the rows are 16-byte aligned, each thread handles
// 16 bytes of gate and of up at a time; other sizes take the scalar kernel.
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, int group, long long total) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / F;
  const int f = (int)(idx - t * F);
  const T* row = gu + (size_t)t * 2 * F;
  const int gc = (f / group) * 2 * group + f % group;
  out[idx] = from_f32<T>(silu_mul(to_f32<T>(row[gc]), to_f32<T>(row[gc + group])));
}

__global__ void swiglu_vec_bf16_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                       int F, int group, long long total_chunks) {
  pdl_prologue();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_chunks) return;
  const int cpr = F >> 3;                       // 8-element chunks per row
  const long long t = idx / cpr;
  const int c = (int)(idx - t * cpr);
  const __nv_bfloat16* row = gu + (size_t)t * 2 * F;
  const int gc = (c * 8 / group) * 2 * group + c * 8 % group;
  const uint4 g = *reinterpret_cast<const uint4*>(row + gc);
  const uint4 u = *reinterpret_cast<const uint4*>(row + gc + group);
  const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
  const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint4 r;
  __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(gh[i]), b = __bfloat1622float2(uh[i]);
    rh[i] = __floats2bfloat162_rn(silu_mul(a.x, b.x), silu_mul(a.y, b.y));
  }
  *reinterpret_cast<uint4*>(out + (size_t)t * F + c * 8) = r;
}

__global__ void swiglu_vec_f32_kernel(const float* __restrict__ gu, float* __restrict__ out, int F, int group,
                                      long long total_chunks) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total_chunks) return;
  const int cpr = F >> 2;
  const long long t = idx / cpr;
  const int c = (int)(idx - t * cpr);
  const float* row = gu + (size_t)t * 2 * F;
  const int gc = (c * 4 / group) * 2 * group + c * 4 % group;
  const float4 g = *reinterpret_cast<const float4*>(row + gc);
  const float4 u = *reinterpret_cast<const float4*>(row + gc + group);
  *reinterpret_cast<float4*>(out + (size_t)t * F + c * 4) =
      make_float4(silu_mul(g.x, u.x), silu_mul(g.y, u.y), silu_mul(g.z, u.z), silu_mul(g.w, u.w));
}

SI_EXPORT int si_swiglu(const void* gu, void* out, int dtype, int num_tokens, int F, int group,
                        cudaStream_t stream) {
  const long long total = (long long)num_tokens * F;
  if (total <= 0) return 0;
  if (group <= 0 || F % group) return -2;
  const int threads = 256;
  const bool aligned = ((uintptr_t)gu % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (dtype == SI_BF16 && aligned && group % 8 == 0) {
    const long long chunks = total / 8;
    si_launch(swiglu_vec_bf16_kernel, dim3((unsigned)((chunks + threads - 1) / threads)), dim3(threads), 0, stream,
              (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, F, group, chunks);
  } else if (dtype == SI_F32 && aligned && group % 4 == 0) {
    const long long chunks = total / 4;
    swiglu_vec_f32_kernel<<<(unsigned)((chunks + threads - 1) / threads), threads, 0, stream>>>(
        (const float*)gu, (float*)out, F, group, chunks);
  } else {
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == SI_BF16)
      swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, F, group, total);
    else
      swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, F, group, total);
  }
  return si_last_error();
}
