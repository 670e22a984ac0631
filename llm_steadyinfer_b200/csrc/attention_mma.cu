// bf16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, fp32
// accumulation, fp32 online softmax), for prompt portions and for decode rows.
//
// A work item is a run of consecutive query tokens of one sequence; a block handles one item
// for one KV head. The G = H / KV query heads that share the KV head are packed into the row
// dimension of the tile (row r = token r / G, head r % G), so a K/V tile is fetched once for all
// of them. K/V tiles come from the pages through cp.async into XOR-swizzled shared memory, two
// stages deep; rows beyond the item's last position, and head-size padding, are zero-filled.
//
//   portion kernel  rows are split over the warps (16 rows each); every warp walks all keys.
//   decode kernel   16*MT rows shared by all warps; the 64 keys of a tile are split over the 4
//                   warps, whose partial (max, sum, acc) are merged at the end. The key range can
//                   also be split over gridDim.z blocks, which write fp32 partials; the block that
//                   finishes last merges them (the reference's split kernel and combine,
//                   src/source/op/kernels/cuda/paged_kernels.cu:96-253, work on one (token, head,
//                   split) per block with scalar fp32 code and no sharing between the heads of a group).
//
// Masking: key j is visible to a row at position p when j <= p and (window == 0 or j > p - window).
#include "attention_common.cuh"

// Shared-memory tile of rows x HS_PAD bf16, 16-byte chunks XOR-swizzled by the row.
template <int HS_PAD>
__device__ __forceinline__ bf16* tile_ptr(bf16* base, int row, int chunk) {
  constexpr int CH = HS_PAD / 8;
  return base + ((size_t)row * CH + (chunk ^ (row & 7))) * 8;
}

// Fetch keys [j0, j0 + ROWS) of one KV head into Ks and Vs. Keys at or beyond kv_end, before 0,
// or on a bad page are zero-filled.
template <int HS_PAD, int ROWS, int THREADS>
__device__ __forceinline__ void load_kv_tile(const AttnParams& p, const int* table, int g, int j0, int kv_lo,
                                             int kv_end, bf16* Ks, bf16* Vs) {
  constexpr int CH = HS_PAD / 8;
  constexpr int TOTAL = ROWS * CH;
  static_assert(TOTAL % THREADS == 0, "tile chunks must divide over the threads");
  const int hs_chunks = p.hs / 8;
#pragma unroll
  for (int it = 0; it < TOTAL / THREADS; ++it) {
    const int id = threadIdx.x + it * THREADS;
    const int row = id / CH, c = id % CH;
    const int j = j0 + row;
    bool valid = j >= kv_lo && j < kv_end && c < hs_chunks;
    size_t off = 0;
    if (valid) {
      const int slot = j / p.page_size;
      const int page = slot < p.table_width ? table[slot] : -1;
      if (page < 0 || page >= p.num_pages) {
        set_status(p.status, SI_BAD_PAGE);
        valid = false;
      } else {
        off = (((size_t)page * p.KV + g) * p.page_size + (j - slot * p.page_size)) * p.hs + c * 8;
      }
    }
    cp_async16(tile_ptr<HS_PAD>(Ks, row, c), p.k_cache + off, valid);
    cp_async16(tile_ptr<HS_PAD>(Vs, row, c), p.v_cache + off, valid);
  }
}

// Fetch the query rows of an item: tile row r is token r / G, head g*G + r % G.
template <int HS_PAD, int ROWS, int THREADS>
__device__ __forceinline__ void load_q_tile(const AttnParams& p, const AttnItem& item, int g, bf16* Qs) {
  constexpr int CH = HS_PAD / 8;
  constexpr int TOTAL = ROWS * CH;
  const int hs_chunks = p.hs / 8;
  for (int id = threadIdx.x; id < TOTAL; id += THREADS) {
    const int row = id / CH, c = id % CH;
    const int tok = row / p.G, hh = row - tok * p.G;
    const bool valid = tok < item.ntok && c < hs_chunks;
    const bf16* src = p.q;
    if (valid) src = p.q + (size_t)(item.row0 + tok) * p.q_stride + (size_t)(g * p.G + hh) * p.hs + c * 8;
    cp_async16(tile_ptr<HS_PAD>(Qs, row, c), src, valid);
  }
}

// ================================ portion kernel ==============================================
template <int HS_PAD, int NWARPS, int BLOCK_N>
__global__ void __launch_bounds__(NWARPS * 32)
attn_portion_kernel(const AttnParams p) {
  constexpr int BLOCK_M = NWARPS * 16;
  constexpr int THREADS = NWARPS * 32;
  constexpr int KT = HS_PAD / 16;          // k steps of Q.K^T
  constexpr int NT = BLOCK_N / 8;          // score n-tiles
  constexpr int DT = HS_PAD / 8;           // output n-tiles
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* Ks = Qs + BLOCK_M * HS_PAD;        // [2][BLOCK_N][HS_PAD]
  bf16* Vs = Ks + 2 * BLOCK_N * HS_PAD;

  const AttnItem item = p.items[blockIdx.x];
  if (item.ntok <= 0) return;
  const int g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (item.seq < 0 || item.seq >= p.num_seqs) {
    if (threadIdx.x == 0) set_status(p.status, SI_BAD_SEQ);
    return;
  }
  const int* table = p.block_table + (size_t)item.seq * p.table_width;
  const int kv_end = item.pos0 + item.ntok;
  const int kv_lo = window_first_key(item.pos0, p.window);
  const int kv_begin = kv_lo / BLOCK_N * BLOCK_N;
  const int ntiles = (kv_end - kv_begin + BLOCK_N - 1) / BLOCK_N;

  load_q_tile<HS_PAD, BLOCK_M, THREADS>(p, item, g, Qs);
  load_kv_tile<HS_PAD, BLOCK_N, THREADS>(p, table, g, kv_begin, kv_lo, kv_end, Ks, Vs);
  cp_async_commit();

  // the two rows this thread owns in the warp's 16-row slab
  const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const int tok_lo = r_lo / p.G, tok_hi = r_hi / p.G;
  const int pos_lo = tok_lo < item.ntok ? item.pos0 + tok_lo : -1;     // -1: row unused
  const int pos_hi = tok_hi < item.ntok ? item.pos0 + tok_hi : -1;
  // highest position of any row of this warp: tiles beyond it are skipped
  const int warp_last_tok = min(item.ntok - 1, (warp * 16 + 15) / p.G);
  const int warp_first_tok = (warp * 16) / p.G;
  const bool warp_active = warp_first_tok < item.ntok;
  const int warp_max_pos = item.pos0 + warp_last_tok;
  const int warp_min_pos = item.pos0 + warp_first_tok;

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int t = 0; t < ntiles; ++t) {
    const int j0 = kv_begin + t * BLOCK_N;
    bf16* Kt = Ks + (t & 1) * BLOCK_N * HS_PAD;
    bf16* Vt = Vs + (t & 1) * BLOCK_N * HS_PAD;
    if (t + 1 < ntiles) {
      load_kv_tile<HS_PAD, BLOCK_N, THREADS>(p, table, g, j0 + BLOCK_N, kv_lo, kv_end,
                                             Ks + ((t + 1) & 1) * BLOCK_N * HS_PAD,
                                             Vs + ((t + 1) & 1) * BLOCK_N * HS_PAD);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    bool skip = !warp_active || j0 > warp_max_pos;
    if (p.window > 0 && j0 + BLOCK_N - 1 <= warp_min_pos - p.window) skip = true;
    if (!skip) {
      float s[NT][4];
#pragma unroll
      for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KT; ++kk) {
        unsigned a0, a1, a2, a3;
        ldsm_x4(a0, a1, a2, a3, tile_ptr<HS_PAD>(Qs, warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), kk * 2 + (lane >> 4)));
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          unsigned b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, tile_ptr<HS_PAD>(Kt, nt * 8 + (lane & 7) + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
          mma_bf16(s[nt], a0, a1, a2, a3, b0, b1);
          mma_bf16(s[nt + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      // mask, scale, running max
      float mx_lo = m_lo, mx_hi = m_hi;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const int pos = (e < 2) ? pos_lo : pos_hi;
          const bool vis = j <= pos && (p.window <= 0 || j > pos - p.window);
          const float v = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
          s[nt][e] = v;
          if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float base_lo = mx_lo == -INFINITY ? 0.f : mx_lo;
      const float base_hi = mx_hi == -INFINITY ? 0.f : mx_hi;
      const float corr_lo = exp2f(m_lo - base_lo), corr_hi = exp2f(m_hi - base_hi);
      m_lo = mx_lo; m_hi = mx_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - base_lo); s[nt][1] = exp2f(s[nt][1] - base_lo);
        s[nt][2] = exp2f(s[nt][2] - base_hi); s[nt][3] = exp2f(s[nt][3] - base_hi);
        sum_lo += s[nt][0] + s[nt][1];
        sum_hi += s[nt][2] + s[nt][3];
      }
      l_lo = l_lo * corr_lo + sum_lo;
      l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        o[i][0] *= corr_lo; o[i][1] *= corr_lo; o[i][2] *= corr_hi; o[i][3] *= corr_hi;
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
        const unsigned a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        const unsigned a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        const unsigned a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        const unsigned a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dt = 0; dt < DT; dt += 2) {
          unsigned b0, b1, b2, b3;
          ldsm_x4_t(b0, b1, b2, b3, tile_ptr<HS_PAD>(Vt, kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dt + (lane >> 4)));
          mma_bf16(o[dt], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[dt + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncthreads();       // everyone is done with this stage before it is refilled
  }
  // row sums over the quad, normalise, store
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r_hi : r_lo;
    const int tok = r / p.G, hh = r - tok * p.G;
    if (tok >= item.ntok) continue;
    bf16* dst = p.out + (size_t)(item.row0 + tok) * p.out_stride + (size_t)(g * p.G + hh) * p.hs;
    const float inv = half ? inv_hi : inv_lo;
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
      const int d = dt * 8 + (lane & 3) * 2;
      if (d < p.hs)
        *reinterpret_cast<__nv_bfloat162*>(dst + d) =
            __floats2bfloat162_rn(o[dt][half * 2] * inv, o[dt][half * 2 + 1] * inv);
    }
  }
}

// ================================ decode kernel ===============================================
// All warps share the 16*MT rows; warp w takes keys [16w, 16w+16) of every 64-key tile. Tiles
// flow through a ring of STAGES shared-memory buffers filled by cp.async.
// With nsplit > 1 each block writes its partial result to scratch and takes a ticket; the block
// that draws the last ticket of its (item, kv head) merges all partials and resets the counter,
// so the merge needs no launch of its own and nobody waits for anybody.
template <int HS_PAD, int MT, int STAGES>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const AttnParams p) {
  constexpr int NWARPS = 4, THREADS = 128, BLOCK_N = 64, ROWS = 16 * MT;
  constexpr int KT = HS_PAD / 16, DT = HS_PAD / 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int s_last;
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* Ks = Qs + ROWS * HS_PAD;                    // [STAGES][BLOCK_N][HS_PAD]
  bf16* Vs = Ks + STAGES * BLOCK_N * HS_PAD;

  const AttnItem item = p.items[blockIdx.x];
  if (item.ntok <= 0) return;
  const int g = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (item.seq < 0 || item.seq >= p.num_seqs) {
    if (threadIdx.x == 0) set_status(p.status, SI_BAD_SEQ);
    return;
  }
  const int* table = p.block_table + (size_t)item.seq * p.table_width;
  const int kv_end_all = item.pos0 + item.ntok;
  const int kv_lo = window_first_key(item.pos0, p.window);
  const int kv_begin_all = kv_lo / BLOCK_N * BLOCK_N;
  // this block's share of the key range, in whole tiles
  const int tiles_all = (kv_end_all - kv_begin_all + BLOCK_N - 1) / BLOCK_N;
  const int tiles_per = (tiles_all + p.nsplit - 1) / p.nsplit;
  const int t_begin = split * tiles_per;
  const int t_end = min(tiles_all, t_begin + tiles_per);
  const int ntiles = max(0, t_end - t_begin);
  const int kv_begin = kv_begin_all + t_begin * BLOCK_N;
  const int kv_end = min(kv_end_all, kv_begin_all + t_end * BLOCK_N);

  float o[MT][DT][4];
  float m[MT][2], l[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m[mt][0] = m[mt][1] = -INFINITY; l[mt][0] = l[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < DT; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
  }
  int pos_of[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      const int r = mt * 16 + (lane >> 2) + 8 * h2;
      const int tok = r / p.G;
      pos_of[mt][h2] = tok < item.ntok ? item.pos0 + tok : -1;
    }

  if (ntiles > 0) load_q_tile<HS_PAD, ROWS, THREADS>(p, item, g, Qs);
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < ntiles)
      load_kv_tile<HS_PAD, BLOCK_N, THREADS>(p, table, g, kv_begin + st * BLOCK_N, kv_lo, kv_end,
                                             Ks + st * BLOCK_N * HS_PAD, Vs + st * BLOCK_N * HS_PAD);
    cp_async_commit();
  }
  for (int t = 0; t < ntiles; ++t) {
    const int j0 = kv_begin + t * BLOCK_N;
    const int stage = t % STAGES;
    bf16* Kt = Ks + stage * BLOCK_N * HS_PAD;
    bf16* Vt = Vs + stage * BLOCK_N * HS_PAD;
    {
      const int tn = t + STAGES - 1;            // refill the buffer that was read in iteration t - 1
      if (tn < ntiles)
        load_kv_tile<HS_PAD, BLOCK_N, THREADS>(p, table, g, kv_begin + tn * BLOCK_N, kv_lo, kv_end,
                                               Ks + (tn % STAGES) * BLOCK_N * HS_PAD,
                                               Vs + (tn % STAGES) * BLOCK_N * HS_PAD);
      cp_async_commit();
    }
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const int jw = j0 + warp * 16;          // this warp's 16 keys
    if (jw < kv_end) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KT; ++kk) {
          unsigned a0, a1, a2, a3, b0, b1, b2, b3;
          ldsm_x4(a0, a1, a2, a3, tile_ptr<HS_PAD>(Qs, mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), kk * 2 + (lane >> 4)));
          ldsm_x4(b0, b1, b2, b3, tile_ptr<HS_PAD>(Kt, warp * 16 + (lane & 7) + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
          mma_bf16(s[0], a0, a1, a2, a3, b0, b1);
          mma_bf16(s[1], a0, a1, a2, a3, b2, b3);
        }
        float mx[2] = {m[mt][0], m[mt][1]};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = jw + nt * 8 + (lane & 3) * 2 + (e & 1);
            const int pos = pos_of[mt][e >> 1];
            const bool vis = j <= pos && (p.window <= 0 || j > pos - p.window);
            const float v = vis ? s[nt][e] * p.scale_log2 : -INFINITY;
            s[nt][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
          }
        float corr[2], base[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
          mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
          base[h2] = mx[h2] == -INFINITY ? 0.f : mx[h2];
          corr[h2] = exp2f(m[mt][h2] - base[h2]);
          m[mt][h2] = mx[h2];
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[nt][e] = exp2f(s[nt][e] - base[e >> 1]);
            sum[e >> 1] += s[nt][e];
          }
        l[mt][0] = l[mt][0] * corr[0] + sum[0];
        l[mt][1] = l[mt][1] * corr[1] + sum[1];
        const unsigned a0 = pack_bf16(s[0][0], s[0][1]), a1 = pack_bf16(s[0][2], s[0][3]);
        const unsigned a2 = pack_bf16(s[1][0], s[1][1]), a3 = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dt = 0; dt < DT; dt += 2) {
          o[mt][dt][0] *= corr[0]; o[mt][dt][1] *= corr[0]; o[mt][dt][2] *= corr[1]; o[mt][dt][3] *= corr[1];
          o[mt][dt + 1][0] *= corr[0]; o[mt][dt + 1][1] *= corr[0]; o[mt][dt + 1][2] *= corr[1]; o[mt][dt + 1][3] *= corr[1];
          unsigned b0, b1, b2, b3;
          ldsm_x4_t(b0, b1, b2, b3, tile_ptr<HS_PAD>(Vt, warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dt + (lane >> 4)));
          mma_bf16(o[mt][dt], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[mt][dt + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // merge the warps: shared memory is free now. fm/fl [NWARPS][ROWS], fo [NWARPS][ROWS][HS_PAD + 4]
  float* fm = reinterpret_cast<float*>(smem_raw);
  float* fl = fm + NWARPS * ROWS;
  float* fo = fl + NWARPS * ROWS;
  constexpr int OS = HS_PAD + 4;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      float lv = l[mt][h2];
      lv += __shfl_xor_sync(0xffffffffu, lv, 1);
      lv += __shfl_xor_sync(0xffffffffu, lv, 2);
      const int r = mt * 16 + (lane >> 2) + 8 * h2;
      if ((lane & 3) == 0) { fm[warp * ROWS + r] = m[mt][h2]; fl[warp * ROWS + r] = lv; }
#pragma unroll
      for (int dt = 0; dt < DT; ++dt) {
        const int d = dt * 8 + (lane & 3) * 2;
        fo[((size_t)warp * ROWS + r) * OS + d] = o[mt][dt][h2 * 2];
        fo[((size_t)warp * ROWS + r) * OS + d + 1] = o[mt][dt][h2 * 2 + 1];
      }
    }
  __syncthreads();
  const int rows_used = min(ROWS, item.ntok * p.G);
  const size_t slab0 = ((size_t)blockIdx.x * p.KV + g) * p.nsplit * ROWS;
  for (int idx = threadIdx.x; idx < rows_used * p.hs; idx += THREADS) {
    const int r = idx / p.hs, d = idx - r * p.hs;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, fm[w * ROWS + r]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float mw = fm[w * ROWS + r];
      const float wgt = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += fl[w * ROWS + r] * wgt;
      acc += fo[((size_t)w * ROWS + r) * OS + d] * wgt;
    }
    if (p.nsplit == 1) {
      const int tok = r / p.G, hh = r - tok * p.G;
      p.out[(size_t)(item.row0 + tok) * p.out_stride + (size_t)(g * p.G + hh) * p.hs + d] =
          __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      const size_t slab = slab0 + (size_t)split * ROWS + r;
      __stcg(p.part_o + slab * p.hs + d, acc);
      if (d == 0) { __stcg(p.part_ml + slab * 2, M); __stcg(p.part_ml + slab * 2 + 1, L); }
    }
  }
  if (p.nsplit == 1) return;

  // ticket: the last block of this (item, kv head) merges the splits
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(p.counters + blockIdx.x * p.KV + g, 1);
    s_last = ticket == p.nsplit - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < rows_used * p.hs; idx += THREADS) {
    const int r = idx / p.hs, d = idx - r * p.hs;
    float M = -INFINITY;
#pragma unroll 8                   // several loads in flight, not one trip to L2 after the other
    for (int s = 0; s < p.nsplit; ++s) M = fmaxf(M, __ldcg(p.part_ml + (slab0 + (size_t)s * ROWS + r) * 2));
    float L = 0.f, acc = 0.f;
#pragma unroll 4
    for (int s = 0; s < p.nsplit; ++s) {
      const size_t slab = slab0 + (size_t)s * ROWS + r;
      const float ms = __ldcg(p.part_ml + slab * 2);
      const float wgt = ms == -INFINITY ? 0.f : exp2f(ms - M);
      L += __ldcg(p.part_ml + slab * 2 + 1) * wgt;
      acc += __ldcg(p.part_o + slab * p.hs + d) * wgt;
    }
    const int tok = r / p.G, hh = r - tok * p.G;
    p.out[(size_t)(item.row0 + tok) * p.out_stride + (size_t)(g * p.G + hh) * p.hs + d] =
        __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x * p.KV + g] = 0;      // ready for the next launch
}

// ---- host side --------------------------------------------------------------------------------
template <typename K>
static int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

static bool fill_params(AttnParams& p, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                        const int* block_table, int table_width, const void* items, void* out, long long out_stride,
                        int num_pages, int page_size, int num_seqs, int H, int KV, int hs, float scale, int window,
                        int* status) {
  if (hs <= 0 || hs % 16 || hs > 256 || KV <= 0 || H % KV || page_size <= 0) return false;
  if ((q_stride % 8) || (out_stride % 2)) return false;          // 16-byte chunks of q, bf16 pairs of out
  p.q = (const bf16*)q; p.q_stride = q_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.block_table = block_table; p.table_width = table_width;
  p.items = (const AttnItem*)items;
  p.out = (bf16*)out; p.out_stride = out_stride;
  p.part_o = nullptr; p.part_ml = nullptr; p.counters = nullptr;
  p.num_pages = num_pages; p.page_size = page_size; p.num_seqs = num_seqs;
  p.H = H; p.KV = KV; p.G = H / KV; p.hs = hs;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window; p.nsplit = 1; p.status = status;
  return true;
}

// Tokens of one item in the portion kernel: floor(rows / G), rows = 64 (head sizes above 128) or 128.
SI_EXPORT int si_attn_portion_tokens(int H, int KV, int hs) {
  const int G = H / KV;
  const int rows = hs > 128 ? 64 : 128;
  return G <= rows ? rows / G : 0;
}

template <int HS_PAD, int NWARPS>
static int launch_portion(const AttnParams& p, int num_items, cudaStream_t stream) {
  constexpr int BLOCK_N = 64;
  const size_t smem = (size_t)(NWARPS * 16 + 4 * BLOCK_N) * HS_PAD * sizeof(bf16);
  auto k = attn_portion_kernel<HS_PAD, NWARPS, BLOCK_N>;
  int rc = set_smem(k, smem);
  if (rc) return rc;
  k<<<dim3(num_items, p.KV), NWARPS * 32, smem, stream>>>(p);
  return si_last_error();
}

// Items are runs of at most si_attn_portion_tokens() tokens.
SI_EXPORT int si_attn_portion(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                              const int* block_table, int table_width, const void* items, int num_items,
                              void* out, long long out_stride, int num_pages, int page_size, int num_seqs,
                              int H, int KV, int hs, float scale, int window, int* status, cudaStream_t stream) {
  if (num_items <= 0) return 0;
  AttnParams p;
  if (!fill_params(p, q, q_stride, k_cache, v_cache, block_table, table_width, items, out, out_stride, num_pages,
                   page_size, num_seqs, H, KV, hs, scale, window, status)) return -2;
  if (si_attn_portion_tokens(H, KV, hs) <= 0) return -2;
  if (hs <= 64) return launch_portion<64, 8>(p, num_items, stream);
  if (hs <= 128) return launch_portion<128, 8>(p, num_items, stream);
  return launch_portion<256, 4>(p, num_items, stream);
}

// Rows a decode item may have (tokens * G): 16, 32 or 64, bounded by the registers the
// accumulators take (rows * head size <= 64 * 64); 0 when G does not fit, and such items go to
// the portion kernel.
SI_EXPORT int si_attn_decode_rows(int H, int KV, int hs) {
  const int G = H / KV;
  const int cap = hs <= 64 ? 64 : (hs <= 128 ? 32 : 16);
  const int need = G <= 16 ? 16 : (G <= 32 ? 32 : 64);
  return (G <= 64 && need <= cap) ? need : 0;
}

// Scratch of the split decode kernel in 4-byte words: SI_ATTN_TICKETS ticket counters (one per (item,
// kv head) is used), then partial outputs and (max, sum) pairs. The tickets must be zero before
// their first use; the kernel leaves them at zero.
SI_EXPORT long long si_attn_decode_scratch_floats(int num_items, int H, int KV, int hs, int nsplit) {
  if (nsplit <= 1) return 0;
  const long long rows = si_attn_decode_rows(H, KV, hs);
  return SI_ATTN_TICKETS + (long long)num_items * KV * nsplit * rows * (hs + 2);
}

template <int HS_PAD> constexpr int decode_stages() { return HS_PAD <= 128 ? 3 : 2; }

// Dynamic shared memory of the decode kernel: the q rows and the K/V stages, or the merge's staging if larger.
template <int HS_PAD, int MT>
constexpr size_t decode_smem_bytes() {
  constexpr int ROWS = 16 * MT;
  constexpr size_t tiles = (size_t)(ROWS + 2 * decode_stages<HS_PAD>() * 64) * HS_PAD * sizeof(bf16);
  constexpr size_t merge = (size_t)4 * ROWS * (2 + HS_PAD + 4) * sizeof(float);
  return merge > tiles ? merge : tiles;
}

template <int HS_PAD, int MT>
static int launch_decode(AttnParams& p, int num_items, cudaStream_t stream) {
  constexpr int STAGES = decode_stages<HS_PAD>();
  const size_t smem = decode_smem_bytes<HS_PAD, MT>();
  auto k = attn_decode_kernel<HS_PAD, MT, STAGES>;
  int rc = set_smem(k, smem);
  if (rc) return rc;
  k<<<dim3(num_items, p.KV, p.nsplit), 128, smem, stream>>>(p);
  return si_last_error();
}

// Items hold at most si_attn_decode_rows() / G tokens. With nsplit > 1, `scratch` holds
// si_attn_decode_scratch_floats() floats.
SI_EXPORT int si_attn_decode(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                             const int* block_table, int table_width, const void* items, int num_items,
                             void* out, long long out_stride, int num_pages, int page_size, int num_seqs,
                             int H, int KV, int hs, float scale, int window, int nsplit, float* scratch,
                             int* status, cudaStream_t stream) {
  if (num_items <= 0) return 0;
  AttnParams p;
  if (!fill_params(p, q, q_stride, k_cache, v_cache, block_table, table_width, items, out, out_stride, num_pages,
                   page_size, num_seqs, H, KV, hs, scale, window, status)) return -2;
  const int rows = si_attn_decode_rows(H, KV, hs);
  if (rows <= 0 || nsplit < 1 || nsplit > 65535) return -2;
  p.nsplit = nsplit;
  if (nsplit > 1) {
    if (!scratch || (long long)num_items * KV > SI_ATTN_TICKETS) return -2;
    p.counters = reinterpret_cast<int*>(scratch);
    p.part_o = scratch + SI_ATTN_TICKETS;
    p.part_ml = p.part_o + (size_t)num_items * KV * nsplit * rows * hs;
  }
  if (hs <= 64) {
    if (rows == 16) return launch_decode<64, 1>(p, num_items, stream);
    if (rows == 32) return launch_decode<64, 2>(p, num_items, stream);
    return launch_decode<64, 4>(p, num_items, stream);
  }
  if (hs <= 128) {
    if (rows == 16) return launch_decode<128, 1>(p, num_items, stream);
    return launch_decode<128, 2>(p, num_items, stream);
  }
  return launch_decode<256, 1>(p, num_items, stream);
}
