// Rotary position encoding fused with the write of K and V into the paged cache.
// One or more blocks per token row of the fused projection output
//   row = [ q: H*hs | k: KV*hs | v: KV*hs ]            (row stride given in elements)
// q is rotated in place; k is rotated and stored, v is stored, at
//   cache[page = table[seq, pos / page_size]][kv head][pos % page_size][:]
// Pairing is rotate-half: (x[i], x[i + rot/2]) for i < rot/2, as in the reference
// (src/source/op/kernels/cuda/rope_kernel.cu:113-148); the angle pos * inv_freq[i],
// its sine and cosine are fp32. The reference's page write
// (paged_kernels.cu:53-89) derives the in-page offset from the physical page id;
// the offset here is pos % page_size. inv_freq == nullptr stores k unrotated.
#include "common.cuh"

// Block (t, hb) handles heads [hb * hpb, (hb + 1) * hpb) of token t, counted over the q heads,
// then the k heads, then the v heads; the host picks hpb so that few rows still fill the GPU.
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, long long row_stride,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ row_seq,
                                     const float* __restrict__ inv_freq, int rot_dim,
                                     const int* __restrict__ block_table, int table_width,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     int num_pages, int page_size, int num_seqs, int H, int KV,
                                     int hs, int hpb, int* status) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int seq = row_seq[t];
  T* row = qkv + (size_t)t * row_stride;
  const int head_begin = blockIdx.y * hpb;
  const int head_end = min(H + 2 * KV, head_begin + hpb);

  long long page = -1;
  if (k_cache && head_end > H) {
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
  const int half = (inv_freq ? rot_dim : 0) / 2;
  const int rot = 2 * half;
  const float fpos = (float)pos;

  // rotated pairs of the q heads (in place) and the k heads (to the cache)
  const int rot_end = min(head_end, H + KV);
  for (int idx = threadIdx.x; idx < (rot_end - head_begin) * half; idx += blockDim.x) {
    const int head = head_begin + idx / half, i = idx % half;
    float s, c;
    sincosf(fpos * inv_freq[i], &s, &c);
    T* x = row + (size_t)head * hs;
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
  const int rest = hs - rot;
  const int k_begin = max(head_begin, H), k_end = rot_end;
  for (int idx = threadIdx.x; idx < (k_end - k_begin) * rest; idx += blockDim.x) {
    const int g = k_begin - H + idx / rest, c = rot + idx % rest;
    k_cache[(((size_t)page * KV + g) * page_size + off) * hs + c] = row[(size_t)(H + g) * hs + c];
  }
  const int v_begin = max(head_begin, H + KV);
  for (int idx = threadIdx.x; idx < (head_end - v_begin) * hs; idx += blockDim.x) {
    const int g = v_begin - H - KV + idx / hs, c = idx % hs;
    v_cache[(((size_t)page * KV + g) * page_size + off) * hs + c] = row[(size_t)(H + KV + g) * hs + c];
  }
}

// bf16 with 16-byte accesses: thread (head lane, chunk c) owns elements [8c, 8c+8) of the first
// and of the second half of the rotated part; it forms the 8 sines and cosines once and walks
// its heads with them. Same block-to-heads mapping as the scalar kernel.
__global__ void rope_kv_write_vec_kernel(__nv_bfloat16* __restrict__ qkv, long long row_stride,
                                         const int* __restrict__ positions, const int* __restrict__ row_seq,
                                         const float* __restrict__ inv_freq, int rot_dim,
                                         const int* __restrict__ block_table, int table_width,
                                         __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                         int num_pages, int page_size, int num_seqs, int H, int KV, int hs,
                                         int hpb, int* status, int trigger) {
  typedef __nv_bfloat16 T;
  if (trigger) pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int seq = row_seq[t];
  T* row = qkv + (size_t)t * row_stride;
  const int head_begin = blockIdx.y * hpb;
  const int head_end = min(H + 2 * KV, head_begin + hpb);
  long long page = -1;
  if (k_cache && head_end > H) {
    if (seq < 0) {
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
  const int cpr = half / 8;                       // chunks per half
  const int lanes_h = blockDim.x / cpr;           // head lanes
  const int c = threadIdx.x % cpr, hl = threadIdx.x / cpr;
  const int rot_end = min(head_end, H + KV);
  // the sines and cosines of the token's angles, once for the block (every head lane needs the same ones)
  __shared__ float s_sin[128], s_cos[128];
  if (head_begin < rot_end) {
    const float fpos = (float)pos;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(fpos * inv_freq[i], &s_sin[i], &s_cos[i]);
  }
  __syncthreads();
  if (hl < lanes_h && head_begin + hl < rot_end) {
    float sn[8], cs[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { sn[i] = s_sin[c * 8 + i]; cs[i] = s_cos[c * 8 + i]; }
    for (int head = head_begin + hl; head < rot_end; head += lanes_h) {
      T* x = row + (size_t)head * hs;
      uint4 lo = *reinterpret_cast<const uint4*>(x + c * 8);
      uint4 hi = *reinterpret_cast<const uint4*>(x + half + c * 8);
      __nv_bfloat162* l2 = reinterpret_cast<__nv_bfloat162*>(&lo);
      __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(l2[i]), b = __bfloat1622float2(h2[i]);
        l2[i] = __floats2bfloat162_rn(a.x * cs[2 * i] - b.x * sn[2 * i], a.y * cs[2 * i + 1] - b.y * sn[2 * i + 1]);
        h2[i] = __floats2bfloat162_rn(b.x * cs[2 * i] + a.x * sn[2 * i], b.y * cs[2 * i + 1] + a.y * sn[2 * i + 1]);
      }
      if (head < H) {
        *reinterpret_cast<uint4*>(x + c * 8) = lo;
        *reinterpret_cast<uint4*>(x + half + c * 8) = hi;
      } else if (page >= 0) {
        T* dst = k_cache + (((size_t)page * KV + (head - H)) * page_size + off) * hs;
        *reinterpret_cast<uint4*>(dst + c * 8) = lo;
        *reinterpret_cast<uint4*>(dst + half + c * 8) = hi;
      }
    }
  }
  if (page < 0) return;
  // dims of k outside the rotated part (8 at a time), and all of v
  const int rest8 = (hs - rot_dim) / 8, hs8 = hs / 8;
  const int k_begin = max(head_begin, H), k_end = rot_end;
  for (int idx = threadIdx.x; idx < (k_end - k_begin) * rest8; idx += blockDim.x) {
    const int g = k_begin - H + idx / rest8, cc = rot_dim + (idx % rest8) * 8;
    *reinterpret_cast<uint4*>(k_cache + (((size_t)page * KV + g) * page_size + off) * hs + cc) =
        *reinterpret_cast<const uint4*>(row + (size_t)(H + g) * hs + cc);
  }
  const int v_begin = max(head_begin, H + KV);
  for (int idx = threadIdx.x; idx < (head_end - v_begin) * hs8; idx += blockDim.x) {
    const int g = v_begin - H - KV + idx / hs8, cc = (idx % hs8) * 8;
    *reinterpret_cast<uint4*>(v_cache + (((size_t)page * KV + g) * page_size + off) * hs + cc) =
        *reinterpret_cast<const uint4*>(row + (size_t)(H + KV + g) * hs + cc);
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
  const int heads = H + 2 * KV;
  // heads per block: all of them when there are many rows, fewer when rows alone cannot fill the GPU
  int hpb = heads;
  while (hpb > 1 && (long long)num_tokens * ((heads + hpb - 1) / hpb) < 4 * si_sm_count()) hpb = (hpb + 1) / 2;
  const int blocks_y = (heads + hpb - 1) / hpb;
  if (blocks_y > 65535) return -2;
  const int work = hpb * hs / 2;
  const int threads = work >= 2048 ? 256 : (work >= 128 ? 128 : 64);
  dim3 grid(num_tokens, blocks_y);
  const bool vec = dtype == SI_BF16 && inv_freq && rot_dim >= 16 && rot_dim <= 256 && rot_dim % 16 == 0 && hs % 8 == 0 &&
                   row_stride % 8 == 0 && ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) &&
                   ((uintptr_t)v_cache % 16 == 0);
  if (vec) {
    const int cpr = rot_dim / 16;
    int vthreads = 256;
    while (vthreads > 32 && vthreads / cpr > hpb && vthreads / 2 >= cpr) vthreads /= 2;
    if (vthreads < cpr) vthreads = ((cpr + 31) / 32) * 32;
    si_launch(rope_kv_write_vec_kernel, grid, dim3(vthreads), 0, stream,
              (__nv_bfloat16*)qkv, row_stride, positions, row_seq, inv_freq, rot_dim, block_table, table_width,
              (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_pages, page_size, num_seqs, H, KV, hs, hpb, status,
              (int)(si_pdl_trigger_enabled() && num_tokens <= 64));
    return si_last_error();
  }
  if (dtype == SI_BF16)
    rope_kv_write_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (__nv_bfloat16*)qkv, row_stride, positions, row_seq, inv_freq, rot_dim, block_table,
        table_width, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_pages, page_size,
        num_seqs, H, KV, hs, hpb, status);
  else
    rope_kv_write_kernel<float><<<grid, threads, 0, stream>>>(
        (float*)qkv, row_stride, positions, row_seq, inv_freq, rot_dim, block_table, table_width,
        (float*)k_cache, (float*)v_cache, num_pages, page_size, num_seqs, H, KV, hs, hpb, status);
  return si_last_error();
}
