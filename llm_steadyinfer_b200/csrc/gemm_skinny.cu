// Matrix product for few rows (decode): out[m, n] = sum_k x[m, k] * W[n, k], M <= 16, bf16
// inputs, fp32 accumulation, bf16 or fp32 output. At these sizes the product is a stream of the
// weight matrix through the SMs; the reference sends it to cuBLAS like every other product
// (src/source/op/kernels/cuda/matmul_kernel.cu:128-150). Here the weights go from global memory
// straight into the A fragments of mma.sync m16n8k16 (rows of W are the 16 "m" of the
// instruction, the rows of x its 8 "n"), 16 bytes per lane and load, without a pass through
// shared memory:
//   lane (g, t) loads W[n0 + g][k .. k+8) and W[n0 + g + 8][k .. k+8) with k = 32 c + 8 t, and
//   x[g][k .. k+8). The sum over k does not care in which order k is visited, so the 8
//   consecutive k of a lane are fed as logical columns (2t, 2t+1, 2t+8, 2t+9) of two mma steps,
//   the same mapping for A and B.
// A block owns 16 output columns; its warps take the 32-wide k chunks in turn (adjacent warps
// read adjacent 64 bytes of a row) and their partial sums are added in a fixed order.
//
// With SWIGLU the product is the stacked gate/up projection with gates and ups interleaved in
// groups of 8 rows of W, so that a block's 16 columns are 8 gates and the 8 ups that belong to
// them: the block stores out[m, f] = silu(gate) * up (both rounded to bf16 first, as when the
// projection is stored and a second kernel applies the activation) and no second kernel runs.
//
// With ROPE the product is the stacked q/k/v projection of a decode step, and what the position-encoding kernel
// would do next happens in the epilogue: a block's 16 columns are 8 columns of the first half of one head and
// their rotation partners in the second half (rotate-half pairs (i, i + head_dim / 2), as in
// src/source/op/kernels/cuda/rope_kernel.cu:113-148), so one thread holds both elements of a pair of one row. It
// rounds them to bf16 (as the stored projection would be), rotates q and k heads by the row's position (angle,
// sine and cosine in fp32), writes q heads to the output and k and v heads straight into the row's cache page.
#include "common.cuh"

typedef __nv_bfloat16 bf16;

// What the ROPE epilogue needs beside the product's own arguments.
struct SkinnyRope {
  const int* positions;      // [M]
  const int* row_seq;        // [M], -1: a padding row, nothing is stored for it
  const float* inv_freq;     // [head_dim / 2]
  const int* block_table;    // [num_seqs, table_width]
  bf16* k_cache;             // [num_pages, KV, page_size, head_dim] or null (nothing is stored)
  bf16* v_cache;
  int table_width, num_pages, page_size, num_seqs, H, KV, hs;
  int* status;
};

__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename TO> __device__ __forceinline__ void store_out(TO* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ uint4 ld_stream(const bf16* p) {      // weights: read once, keep out of L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_cached(const bf16* p) {      // x: small, shared by every block
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Rows of W or x beyond N or M are replaced by row 0: their products land in output elements
// that are never stored, so the loads need no predicate.
template <int MT, int WARPS, int UNROLL, typename TO, bool SWIGLU = false, bool ROPE = false>
__global__ void __launch_bounds__(WARPS * 32, 512 / (WARPS * 32))
gemm_skinny_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ W, long long ldw,
                   TO* __restrict__ out, long long ldo, int M, int N, int K, int trigger, const SkinnyRope rope) {
  __shared__ float red[WARPS][MT][32][4];
  if (trigger == 1) pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  // the block's 16 rows of W: n0 .. n0+7 and n1 .. n1+7 (next to each other, or a rotation's two halves)
  const int per_head = ROPE ? rope.hs / 16 : 1;
  const int n0 = ROPE ? (blockIdx.x / per_head) * rope.hs + (blockIdx.x % per_head) * 8 : blockIdx.x * 16;
  const int n1 = ROPE ? n0 + rope.hs / 2 : n0 + 8;
  const bf16* w0 = W + (size_t)(n0 + g < N ? n0 + g : 0) * ldw + t * 8;
  const bf16* w1 = W + (size_t)(n1 + g < N ? n1 + g : 0) * ldw + t * 8;
  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;

  const int full = K >> 5;                      // whole 32-wide chunks
  int c = warp;
  const bf16* xr[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) xr[mt] = x + (size_t)(mt * 8 + g < M ? mt * 8 + g : 0) * ldx + t * 8;
  // The weights do not depend on the kernel before this one: the first round of their loads is in flight
  // before this kernel waits for that kernel's results (x).
  if (c + (UNROLL - 1) * WARPS < full) {
    uint4 a_lo[UNROLL], a_hi[UNROLL], xb[UNROLL][MT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (c + u * WARPS) * 32;
      a_lo[u] = ld_stream(w0 + k);
      a_hi[u] = ld_stream(w1 + k);
    }
    pdl_wait();
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (c + u * WARPS) * 32;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) xb[u][mt] = ld_cached(xr[mt] + k);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma16816(acc[mt], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, xb[u][mt].x, xb[u][mt].y);
        mma16816(acc[mt], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, xb[u][mt].z, xb[u][mt].w);
      }
    c += WARPS * UNROLL;
  } else {
    pdl_wait();
  }
  for (; c + (UNROLL - 1) * WARPS < full; c += WARPS * UNROLL) {
    uint4 a_lo[UNROLL], a_hi[UNROLL], xb[UNROLL][MT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (c + u * WARPS) * 32;
      a_lo[u] = ld_stream(w0 + k);
      a_hi[u] = ld_stream(w1 + k);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) xb[u][mt] = ld_cached(xr[mt] + k);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma16816(acc[mt], a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, xb[u][mt].x, xb[u][mt].y);
        mma16816(acc[mt], a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, xb[u][mt].z, xb[u][mt].w);
      }
  }
  if (trigger == 2) pdl_trigger();
  // what is left: whole chunks one at a time, then the part of a chunk (K is a multiple of 8).
  // Lanes past the end load nothing and feed zeros; every lane of the warp issues the same mma
  // (mma.sync must not sit in a divergent branch).
  const int nchunks = (K + 31) >> 5;
  for (; c < nchunks; c += WARPS) {
    const int k = c * 32;
    const bool in = k + t * 8 < K;
    uint4 lo = make_uint4(0, 0, 0, 0), hi = lo, xv[MT];
    if (in) { lo = ld_stream(w0 + k); hi = ld_stream(w1 + k); }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      xv[mt] = make_uint4(0, 0, 0, 0);
      if (in) xv[mt] = ld_cached(xr[mt] + k);
    }
    __syncwarp();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      mma16816(acc[mt], lo.x, hi.x, lo.y, hi.y, xv[mt].x, xv[mt].y);
      mma16816(acc[mt], lo.z, hi.z, lo.w, hi.w, xv[mt].z, xv[mt].w);
    }
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int e = 0; e < 4; ++e) red[warp][mt][lane][e] = acc[mt][e];
  __syncthreads();
  if constexpr (ROPE) {
    // threads (mt, lane, e) add the partial sums of the two elements of one rotation pair of one row
    const int head = blockIdx.x / per_head, half = rope.hs / 2;
    for (int idx = threadIdx.x; idx < MT * 32 * 2; idx += WARPS * 32) {
      const int mt = idx / 64, ln = (idx >> 1) & 31, e = idx & 1;
      float a = 0.f, b = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) { a += red[w][mt][ln][e]; b += red[w][mt][ln][e + 2]; }
      const int m = mt * 8 + (ln & 3) * 2 + e;
      if (m >= M) continue;
      const int i = (blockIdx.x % per_head) * 8 + (ln >> 2);       // index in the head's first half
      const float x0 = __bfloat162float(__float2bfloat16_rn(a)), x1 = __bfloat162float(__float2bfloat16_rn(b));
      float y0 = x0, y1 = x1;
      const int pos = rope.positions[m];
      if (head < rope.H + rope.KV) {
        float sn, cs;
        sincosf((float)pos * rope.inv_freq[i], &sn, &cs);
        y0 = x0 * cs - x1 * sn;
        y1 = x1 * cs + x0 * sn;
      }
      if (head < rope.H) {
        bf16* dst = (bf16*)out + (size_t)m * ldo + (size_t)head * rope.hs + i;
        dst[0] = __float2bfloat16_rn(y0);
        dst[half] = __float2bfloat16_rn(y1);
        continue;
      }
      const int seq = rope.row_seq[m];
      if (!rope.k_cache || seq < 0) continue;                      // a layer that stores nothing, or a padding row
      if (seq >= rope.num_seqs) { set_status(rope.status, SI_BAD_SEQ); continue; }
      const int slot = pos / rope.page_size;
      const int page = (pos >= 0 && slot < rope.table_width) ? rope.block_table[(size_t)seq * rope.table_width + slot] : -1;
      if (page < 0 || page >= rope.num_pages) { set_status(rope.status, SI_BAD_PAGE); continue; }
      const bool is_k = head < rope.H + rope.KV;
      const int kvh = head - rope.H - (is_k ? 0 : rope.KV);
      bf16* dst = (is_k ? rope.k_cache : rope.v_cache) +
                  (((size_t)page * rope.KV + kvh) * rope.page_size + pos % rope.page_size) * rope.hs + i;
      dst[0] = __float2bfloat16_rn(y0);
      dst[half] = __float2bfloat16_rn(y1);
    }
  } else if constexpr (SWIGLU) {
    // threads (mt, lane, e) add the partial sums of gate (element e) and up (element e + 2) of one output
    for (int idx = threadIdx.x; idx < MT * 32 * 2; idx += WARPS * 32) {
      const int mt = idx / 64, ln = (idx >> 1) & 31, e = idx & 1;
      float gs = 0.f, us = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) { gs += red[w][mt][ln][e]; us += red[w][mt][ln][e + 2]; }
      const int f = blockIdx.x * 8 + (ln >> 2);
      const int m = mt * 8 + (ln & 3) * 2 + e;
      if (2 * f < N && m < M)
        store_out<TO>(out + (size_t)m * ldo + f, silu_mul(__bfloat162float(__float2bfloat16_rn(gs)), __bfloat162float(__float2bfloat16_rn(us))));
    }
  } else {
    // threads (mt, lane, e) add the warps' partial sums in warp order and store
    for (int idx = threadIdx.x; idx < MT * 32 * 4; idx += WARPS * 32) {
      const int mt = idx / 128, ln = (idx >> 2) & 31, e = idx & 3;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) s += red[w][mt][ln][e];
      const int n = n0 + (ln >> 2) + ((e >> 1) ? 8 : 0);
      const int m = mt * 8 + (ln & 3) * 2 + (e & 1);
      if (n < N && m < M) store_out<TO>(out + (size_t)m * ldo + n, s);
    }
  }
}

// Eight warps a block (two blocks an SM) unless the blocks would then make more than one round but no more than
// two: with four warps a block, four blocks fit an SM and all of them run at once, sharing the memory bandwidth,
// instead of a full round followed by a part of one.
static inline bool skinny_four_warps(unsigned blocks) {
  const unsigned sms = (unsigned)si_sm_count();
  return blocks > 2 * sms && blocks <= 4 * sms;
}

template <int WARPS, typename TO, bool SWIGLU, bool ROPE>
static void skinny_launch(unsigned blocks, cudaStream_t stream, const bf16* xp, long long ldx, const bf16* wp, long long ldw,
                          TO* out, long long ldo, int M, int N, int K, const SkinnyRope& r) {
  constexpr int UNROLL = 8;
  const int trig = si_pdl_trigger_mode(blocks, (512 / (WARPS * 32)) * si_sm_count());
  if (M <= 8) si_launch(gemm_skinny_kernel<1, WARPS, UNROLL, TO, SWIGLU, ROPE>, dim3(blocks), dim3(WARPS * 32), 0, stream, xp, ldx, wp, ldw, out, ldo, M, N, K, trig, r);
  else si_launch(gemm_skinny_kernel<2, WARPS, UNROLL, TO, SWIGLU, ROPE>, dim3(blocks), dim3(WARPS * 32), 0, stream, xp, ldx, wp, ldw, out, ldo, M, N, K, trig, r);
}

template <typename TO, bool SWIGLU, bool ROPE>
static void skinny_dispatch(unsigned blocks, cudaStream_t stream, const bf16* xp, long long ldx, const bf16* wp, long long ldw,
                            TO* out, long long ldo, int M, int N, int K, const SkinnyRope& r) {
  if (skinny_four_warps(blocks)) skinny_launch<4, TO, SWIGLU, ROPE>(blocks, stream, xp, ldx, wp, ldw, out, ldo, M, N, K, r);
  else skinny_launch<8, TO, SWIGLU, ROPE>(blocks, stream, xp, ldx, wp, ldw, out, ldo, M, N, K, r);
}

// Largest M this kernel takes.
SI_EXPORT int si_gemm_skinny_max_rows() { return 16; }

// out_dtype: SI_BF16 or SI_F32. Returns -2 when the sizes or alignments are not supported.
SI_EXPORT int si_gemm_skinny(const void* x, long long ldx, const void* W, long long ldw, void* out, long long ldo,
                             int out_dtype, int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8)) return -2;
  if (((uintptr_t)x % 16) || ((uintptr_t)W % 16)) return -2;
  const unsigned blocks = (unsigned)((N + 15) / 16);
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)W;
  if (out_dtype == SI_BF16) skinny_dispatch<bf16, false, false>(blocks, stream, xp, ldx, wp, ldw, (bf16*)out, ldo, M, N, K, SkinnyRope());
  else skinny_dispatch<float, false, false>(blocks, stream, xp, ldx, wp, ldw, (float*)out, ldo, M, N, K, SkinnyRope());
  return si_last_error();
}

// out[M, F] = silu(gate) * up of the stacked projection x[M, K] W[2F, K]^T whose rows are interleaved in
// groups of 8 (8 gates, their 8 ups, ...); F a multiple of 8, bf16 output.
SI_EXPORT int si_gemm_skinny_swiglu(const void* x, long long ldx, const void* W, long long ldw, void* out, long long ldo,
                                    int M, int F, int K, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return 0;
  if (M > 16 || K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8) || (F % 8)) return -2;
  if (((uintptr_t)x % 16) || ((uintptr_t)W % 16)) return -2;
  const unsigned blocks = (unsigned)(F / 8);
  skinny_dispatch<bf16, true, false>(blocks, stream, (const bf16*)x, ldx, (const bf16*)W, ldw, (bf16*)out, ldo, M, 2 * F, K, SkinnyRope());
  return si_last_error();
}

// The stacked q/k/v projection of at most 16 rows with the rotation of q and k and the store of k and v into
// the cache pages in its epilogue (see the head of this file): x [M, K], W [(H + 2 KV) * hs, K] with q heads
// first, then k, then v; `out` [M, >= H * hs] bf16 takes the rotated q heads. hs a multiple of 16 with the whole
// head rotated (rot_dim == hs). k_cache / v_cache null: nothing is stored. Returns -2 for what it does not take.
SI_EXPORT int si_gemm_skinny_qkv_rope(const void* x, long long ldx, const void* W, long long ldw, void* out, long long ldo,
                                      int M, int K, const int* positions, const int* row_seq, const float* inv_freq,
                                      const int* block_table, int table_width, void* k_cache, void* v_cache,
                                      int num_pages, int page_size, int num_seqs, int H, int KV, int hs, int* status,
                                      cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > 16 || K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8) || H <= 0 || KV <= 0 || hs <= 0 || (hs % 16)) return -2;
  if (((uintptr_t)x % 16) || ((uintptr_t)W % 16) || !positions || !row_seq || !inv_freq || page_size <= 0) return -2;
  if (k_cache && (!v_cache || !block_table)) return -2;
  const int N = (H + 2 * KV) * hs;
  const unsigned blocks = (unsigned)((H + 2 * KV) * (hs / 16));
  SkinnyRope r;
  r.positions = positions; r.row_seq = row_seq; r.inv_freq = inv_freq; r.block_table = block_table;
  r.k_cache = (bf16*)k_cache; r.v_cache = (bf16*)v_cache;
  r.table_width = table_width; r.num_pages = num_pages; r.page_size = page_size; r.num_seqs = num_seqs;
  r.H = H; r.KV = KV; r.hs = hs; r.status = status;
  skinny_dispatch<bf16, false, true>(blocks, stream, (const bf16*)x, ldx, (const bf16*)W, ldw, (bf16*)out, ldo, M, N, K, r);
  return si_last_error();
}
