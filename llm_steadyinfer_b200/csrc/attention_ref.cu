// Plain attention over the paged cache, one block per (token row, query head), in
// fp32 arithmetic for fp32 or bf16 storage. It is the true-32-bit product path and the
// yardstick the tensor-core kernels are tested against.
//   s_j = scale * q_h . K[j, g],  j in [max(0, pos - window + 1), pos],  g = h / (H / KV)
//   out_h = sum_j softmax(s)_j V[j, g]
// as in the reference's split kernel (src/source/op/kernels/cuda/paged_kernels.cu:96-206)
// and its oracle form (cpu/mha_kernel.cpp:112-171). Causality inside a portion comes from
// all rows' K/V being stored before this kernel runs, each row reading up to its own
// position. The order of the reduction for a row depends only on its position, never on
// the rest of the batch: warp w of 4 walks keys j0+w, j0+w+4, ... with a running max, and
// the four partial results are merged at the end.
#include "common.cuh"
#include <math.h>

#define REF_WARPS 4
#define REF_MAX_PER_LANE 8   // head sizes up to 256

template <typename T>
__global__ void __launch_bounds__(REF_WARPS * 32)
paged_attention_ref_kernel(const T* __restrict__ q, long long q_row_stride,
                           const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                           const int* __restrict__ block_table, int table_width,
                           const int* __restrict__ row_seq, const int* __restrict__ positions,
                           T* __restrict__ out, long long out_row_stride, int num_pages,
                           int page_size, int num_seqs, int H, int KV, int hs, float scale,
                           int window, int* status) {
  extern __shared__ float smem[];   // [REF_WARPS][hs] accumulators, then m[REF_WARPS], l[REF_WARPS]
  const int t = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = h / (H / KV);
  const int pos = positions[t];
  const int seq = row_seq[t];
  T* o = out + (size_t)t * out_row_stride + (size_t)h * hs;
  if (seq < 0 || seq >= num_seqs) {      // seq < 0 marks a padding row of a fixed-shape step
    if (threadIdx.x == 0 && seq >= 0) set_status(status, SI_BAD_SEQ);
    for (int d = threadIdx.x; d < hs; d += blockDim.x) o[d] = from_f32<T>(0.f);
    return;
  }
  const int* table = block_table + (size_t)seq * table_width;
  const T* qh = q + (size_t)t * q_row_stride + (size_t)h * hs;

  float qr[REF_MAX_PER_LANE], acc[REF_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < REF_MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    qr[i] = d < hs ? to_f32<T>(qh[d]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int j0 = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  for (int j = j0 + warp; j <= pos; j += REF_WARPS) {
    const int slot = j / page_size;
    const int page = slot < table_width ? table[slot] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0) set_status(status, SI_BAD_PAGE);
      continue;
    }
    const size_t base = (((size_t)page * KV + g) * page_size + (j - slot * page_size)) * hs;
    const T* kp = k_cache + base;
    const T* vp = v_cache + base;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < REF_MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < hs) dot += qr[i] * to_f32<T>(kp[d]);
    }
    dot = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, dot);
    const float corr = expf(m - m_new);
    const float p = expf(dot - m_new);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < REF_MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < hs) acc[i] = acc[i] * corr + p * to_f32<T>(vp[d]);
    }
    m = m_new;
  }
  float* sacc = smem;
  float* sm = smem + REF_WARPS * hs;
  float* sl = sm + REF_WARPS;
#pragma unroll
  for (int i = 0; i < REF_MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < hs) sacc[warp * hs + d] = acc[i];
  }
  if (lane == 0) { sm[warp] = m; sl[warp] = l; }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < REF_WARPS; ++w) M = fmaxf(M, sm[w]);
  float L = 0.f, wgt[REF_WARPS];
#pragma unroll
  for (int w = 0; w < REF_WARPS; ++w) {
    wgt[w] = sm[w] == -INFINITY ? 0.f : expf(sm[w] - M);
    L += sl[w] * wgt[w];
  }
  for (int d = threadIdx.x; d < hs; d += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < REF_WARPS; ++w) v += sacc[w * hs + d] * wgt[w];
    o[d] = from_f32<T>(L > 0.f ? v / L : 0.f);
  }
}

SI_EXPORT int si_paged_attention_ref(const void* q, int dtype, long long q_row_stride,
                                     const void* k_cache, const void* v_cache,
                                     const int* block_table, int table_width, const int* row_seq,
                                     const int* positions, void* out, long long out_row_stride,
                                     int num_pages, int page_size, int num_tokens, int num_seqs,
                                     int H, int KV, int hs, float scale, int window, int* status,
                                     cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hs > 32 * REF_MAX_PER_LANE || hs <= 0 || KV <= 0 || H % KV) return -2;
  dim3 grid(num_tokens, H);
  const size_t smem = (size_t)(REF_WARPS * hs + 2 * REF_WARPS) * sizeof(float);
  if (dtype == SI_BF16)
    paged_attention_ref_kernel<__nv_bfloat16><<<grid, REF_WARPS * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)k_cache,
        (const __nv_bfloat16*)v_cache, block_table, table_width, row_seq, positions,
        (__nv_bfloat16*)out, out_row_stride, num_pages, page_size, num_seqs, H, KV, hs, scale,
        window, status);
  else
    paged_attention_ref_kernel<float><<<grid, REF_WARPS * 32, smem, stream>>>(
        (const float*)q, q_row_stride, (const float*)k_cache, (const float*)v_cache, block_table,
        table_width, row_seq, positions, (float*)out, out_row_stride, num_pages, page_size,
        num_seqs, H, KV, hs, scale, window, status);
  return si_last_error();
}
