// Rotary position encoding fused with the write of K and V into the paged cache.
// One block per token row of the fused projection output
//   row = [ q: H*hs | k: KV*hs | v: KV*hs ]            (row stride given in elements)
// q is rotated in place; k is rotated and stored, v is stored, at
//   cache[page = table[seq, pos / page_size]][kv head][pos % page_size][:]
// Pairing is rotate-half: (x[i], x[i + rot/2]) for i < rot/2, as in the reference
// (src/source/op/kernels/cuda/rope_kernel.cu:113-148); the angle pos * inv_freq[i],
// its sine and cosine are fp32. The reference's page write
// (paged_kernels.cu:53-89) derives the in-page offset from the physical page id;
// the offset here is pos % page_size. inv_freq == nullptr stores k unrotated.
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, long long row_stride,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ row_seq,
                                     const float* __restrict__ inv_freq, int rot_dim,
                                     const int* __restrict__ block_table, int table_width,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     int num_pages, int page_size, int num_seqs, int H, int KV,
                                     int hs, int* status) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int seq = row_seq[t];
  T* row = qkv + (size_t)t * row_stride;
  T* krow = row + (size_t)H * hs;
  T* vrow = krow + (size_t)KV * hs;

  long long page = -1;
  if (k_cache) {
    if (seq < 0) {
      // a padding row of a fixed-shape step: nothing is stored
    } else if (seq >= num_seqs) {
      if (threadIdx.x == 0) set_status(status, SI_BAD_SEQ);
    } else {
      const int slot = pos / page_size;
      const int p = (pos >= 0 && slot < table_width) ? block_table[(size_t)seq * table_width + slot] : -1;
      if (p < 0 || p >= num_pages) {
        if (threadIdx.x == 0) set_status(status, SI_BAD_PAGE);
      } else {
        page = p;
      }
    }
  }
  const int off = pos % page_size;
  const int half = rot_dim / 2;
  const float fpos = (float)pos;

  // rotated pairs of q heads (in place) and k heads (to the cache)
  const int pairs = inv_freq ? (H + KV) * half : 0;
  for (int idx = threadIdx.x; idx < pairs; idx += blockDim.x) {
    const int head = idx / half, i = idx - head * half;
    float s, c;
    sincosf(fpos * inv_freq[i], &s, &c);
    T* x = head < H ? row + (size_t)head * hs : krow + (size_t)(head - H) * hs;
    const float x0 = to_f32<T>(x[i]), x1 = to_f32<T>(x[i + half]);
    const T y0 = from_f32<T>(x0 * c - x1 * s);
    const T y1 = from_f32<T>(x1 * c + x0 * s);
    if (head < H) {
      x[i] = y0;
      x[i + half] = y1;
    } else if (page >= 0) {
      T* dst = k_cache + (((size_t)page * KV + (head - H)) * page_size + off) * hs;
      dst[i] = y0;
      dst[i + half] = y1;
    }
  }
  if (page < 0) return;
  // dims of k outside the rotated part, and all of v
  const int rot = inv_freq ? rot_dim : 0;
  const int rest = hs - rot;
  for (int idx = threadIdx.x; idx < KV * rest; idx += blockDim.x) {
    const int g = idx / rest, c = rot + (idx - g * rest);
    k_cache[(((size_t)page * KV + g) * page_size + off) * hs + c] = krow[(size_t)g * hs + c];
  }
  for (int idx = threadIdx.x; idx < KV * hs; idx += blockDim.x) {
    const int g = idx / hs, c = idx - g * hs;
    v_cache[(((size_t)page * KV + g) * page_size + off) * hs + c] = vrow[idx];
  }
}

SI_EXPORT int si_rope_kv_write(void* qkv, int dtype, long long row_stride, const int* positions,
                               const int* row_seq, const float* inv_freq, int rot_dim,
                               const int* block_table, int table_width, void* k_cache,
                               void* v_cache, int num_pages, int page_size, int num_tokens,
                               int num_seqs, int H, int KV, int hs, int* status,
                               cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rot_dim < 0 || rot_dim > hs || (rot_dim & 1)) return -2;
  const int work = (H + 2 * KV) * hs / 2;
  const int threads = work >= 2048 ? 256 : 128;
  if (dtype == SI_BF16)
    rope_kv_write_kernel<__nv_bfloat16><<<num_tokens, threads, 0, stream>>>(
        (__nv_bfloat16*)qkv, row_stride, positions, row_seq, inv_freq, rot_dim, block_table,
        table_width, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_pages, page_size,
        num_seqs, H, KV, hs, status);
  else
    rope_kv_write_kernel<float><<<num_tokens, threads, 0, stream>>>(
        (float*)qkv, row_stride, positions, row_seq, inv_freq, rot_dim, block_table, table_width,
        (float*)k_cache, (float*)v_cache, num_pages, page_size, num_seqs, H, KV, hs, status);
  return si_last_error();
}
