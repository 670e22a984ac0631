// Attention for prompt portions on the 5th-generation tensor cores (tcgen05), bf16, over the
// paged cache. One block handles one work item (a run of consecutive query tokens of a sequence)
// for one KV head: 128 rows = tokens x the G query heads of the KV head (row r = token r / G,
// head r % G), against key tiles of 128.
//
//   warp 8 (producer)  looks up the pages of a tile and issues its K and V boxes by TMA
//                      (128-byte swizzle) into one of two stages;
//   warp 9 (issuer)    S = Q K^T with tcgen05.mma into tensor memory (Q, K K-major) and, once the
//                      probabilities are in shared memory, O += P V (V is the MN-major operand, as
//                      it lies in the cache); the next tile's S is issued as soon as the rows of the
//                      current one are in registers, so it runs under the softmax;
//   warps 0-7          two threads per row (warps 0-3 take keys 0-63 of a tile, warps 4-7 keys 64-127):
//                      read the row of S from tensor memory (tcgen05.ld), mask, exchange the row
//                      maximum, softmax in fp32 (exp2 of scale*log2e-scaled scores) against a base
//                      that is raised only when the maximum has grown by more than 2^8 (then the row
//                      of O in tensor memory is rescaled with tcgen05.ld/st), write the bf16
//                      probabilities into the swizzled P tile; at the end read O, divide by the row sum.
//
// The reference computes prompt attention row by row with its scalar split kernel
// (src/source/op/kernels/cuda/paged_kernels.cu:96-206). Conditions here: head_dim 64 or 128, page size
// a power of two from 8 to 64, G <= 128; other layouts use the mma.sync kernel. Every mbarrier wait
// is bounded; when one runs out the block sets SI_WAIT_LIMIT and leaves without storing.
#include "attention_common.cuh"
#include "tma_common.cuh"

// 2^x in fp32 by the hardware approximation (2 ulp); exp2(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int NROWS>
__device__ __forceinline__ bf16* half_ptr(bf16* base, int row, int chunk) {
  return base + (size_t)(chunk >> 3) * (NROWS * 64) + (size_t)row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}

template <int NH>
__global__ void __launch_bounds__(320)
attn_portion_tc05_kernel(const AttnParams p, const __grid_constant__ CUtensorMap kmap,
                         const __grid_constant__ CUtensorMap vmap, int log2_page) {
  constexpr int BM = 128, BN = 128, HS = NH * 64, STAGES = 2;
  constexpr int TILE = NH * BN * 64;                 // elements of a K (or V) tile: NH halves of [128][64]
  constexpr int TM_S = 0, TM_T = BN;                 // tensor-memory columns of S and of T = P V
  constexpr int TM_COLS = 256;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
  __shared__ __align__(8) uint64_t s_full, s_free, p_full, t_full;
  __shared__ unsigned tmem_slot;
  __shared__ int s_abort;
  __shared__ float xmax[2][2][BM];                   // [tile parity][column half][row]: row maxima to exchange
  __shared__ float xsum[2][BM];
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);     // [NH][128][64]
  bf16* Ps = Qs + BM * HS;                           // [2][128][64]   (keys 0-63, 64-127)
  bf16* Ks = Ps + BM * BN;                           // [STAGES][TILE]
  bf16* Vs = Ks + STAGES * TILE;

  // items of a prompt come in order of position, so the last ones have the most keys: start with those
  const AttnItem item = p.items[gridDim.x - 1 - blockIdx.x];
  if (item.ntok <= 0) return;
  const int g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (item.seq < 0 || item.seq >= p.num_seqs) {
    if (threadIdx.x == 0) set_status(p.status, SI_BAD_SEQ);
    return;
  }
  const int* table = p.block_table + (size_t)item.seq * p.table_width;
  const int kv_end = item.pos0 + item.ntok;
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, item.pos0 - p.window + 1) / BN * BN;
  const int ntiles = (kv_end - kv_begin + BN - 1) / BN;
  const int page_rows = 1 << log2_page;
  const int pages_per_tile = BN >> log2_page;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    mbar_init(&s_full, 1);
    mbar_init(&p_full, 8);                           // one arrival per softmax warp
    mbar_init(&s_free, 8);
    mbar_init(&t_full, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 9) tmem_alloc(&tmem_slot, TM_COLS);
  // rows of the last tile that no copy fills must hold finite numbers (they meet zero probabilities)
  if ((kv_end - kv_begin) % BN != 0) {
    const int stage = (ntiles - 1) % STAGES;
    uint4* kz = reinterpret_cast<uint4*>(Ks + (size_t)stage * TILE);
    uint4* vz = reinterpret_cast<uint4*>(Vs + (size_t)stage * TILE);
    for (int i = threadIdx.x; i < TILE / 8; i += blockDim.x) { kz[i] = make_uint4(0, 0, 0, 0); vz[i] = make_uint4(0, 0, 0, 0); }
  }
  // query rows: tile row r is token r / G, head g*G + r % G
  for (int id = threadIdx.x; id < BM * (HS / 8); id += blockDim.x) {
    const int row = id / (HS / 8), c = id % (HS / 8);
    const int tok = row / p.G, hh = row - tok * p.G;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tok < item.ntok)
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(item.row0 + tok) * p.q_stride + (size_t)(g * p.G + hh) * p.hs + c * 8);
    *reinterpret_cast<uint4*>(half_ptr<BM>(Qs, row, c)) = v;
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  tc05_fence_before_sync();
  __syncthreads();
  tc05_fence_after_sync();
  const unsigned tmem = tmem_slot;

  if (warp == 8) {
    // ---- producer: box b = (page, half, K or V) of each tile, boxes spread over the lanes. K and V
    // have barriers of their own: a K stage is free as soon as S has been computed from it, long
    // before the V stage of the same tile, so the next keys arrive under the softmax.
    const int boxes = pages_per_tile * NH * 2;
    for (int t = 0; t < ntiles; ++t) {
      const int stage = t % STAGES;
      const int j = kv_begin + t * BN;
      int cnt = 0;                                   // boxes of K (the same number of V) this lane group fetches
      int page_of[2] = {-1, -1};
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int b = lane + 32 * i;
        const int pg = b / (2 * NH);
        if (b < boxes && j + pg * page_rows < kv_end) {           // pages past the last key are not fetched
          const int slot = (j >> log2_page) + pg;
          int page = slot < p.table_width ? table[slot] : -1;
          if (page < 0 || page >= p.num_pages) { set_status(p.status, SI_BAD_PAGE); page = -1; }
          page_of[i] = page;
          cnt += (page >= 0) && !(b & 1);
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
      bool ok = true;
      if (t >= STAGES) ok = mbar_wait(&k_empty[stage], (unsigned)(((t / STAGES) - 1) & 1));
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) { set_status(p.status, SI_WAIT_LIMIT); s_abort = 1; }
        break;
      }
      if (lane == 0) mbar_expect_tx(&k_full[stage], (unsigned)(cnt * page_rows * 128));
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int b = lane + 32 * i;
        if (page_of[i] < 0 || (b & 1)) continue;
        const int pg = b / (2 * NH), h = (b >> 1) % NH;
        const int row = (page_of[i] * p.KV + g) << log2_page;
        const size_t off = (size_t)stage * TILE + (size_t)h * (BN * 64) + (size_t)(pg * page_rows) * 64;
        tma_load_2d(Ks + off, &kmap, &k_full[stage], h * 64, row);
      }
      if (t >= STAGES) ok = mbar_wait(&v_empty[stage], (unsigned)(((t / STAGES) - 1) & 1));
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) { set_status(p.status, SI_WAIT_LIMIT); s_abort = 1; }
        break;
      }
      if (lane == 0) mbar_expect_tx(&v_full[stage], (unsigned)(cnt * page_rows * 128));
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int b = lane + 32 * i;
        if (page_of[i] < 0 || !(b & 1)) continue;
        const int pg = b / (2 * NH), h = (b >> 1) % NH;
        const int row = (page_of[i] * p.KV + g) << log2_page;
        const size_t off = (size_t)stage * TILE + (size_t)h * (BN * 64) + (size_t)(pg * page_rows) * 64;
        tma_load_2d(Vs + off, &vmap, &v_full[stage], h * 64, row);
      }
    }
  } else if (warp == 9) {
    // ---- issuer: one lane issues the tensor-core instructions
    if (lane == 0) {
      constexpr unsigned idesc_s = umma_idesc_bf16(BM, BN, false);
      constexpr unsigned idesc_t = umma_idesc_bf16(BM, HS, true);
      auto issue_s = [&](int t) {       // S[128, 128] = Q[128, HS] K_t[128 keys, HS]^T: 4 steps per 64-column half
        const int stage = t % STAGES;
#pragma unroll
        for (int kk = 0; kk < HS / 16; ++kk) {
          const unsigned long long qd = umma_desc_sw128(Qs + (size_t)(kk >> 2) * (BM * 64), 16, 1024) + 2 * (kk & 3);
          const unsigned long long kd = umma_desc_sw128(Ks + (size_t)stage * TILE + (size_t)(kk >> 2) * (BN * 64), 16, 1024) + 2 * (kk & 3);
          tc05_mma_bf16(tmem + TM_S, qd, kd, idesc_s, kk != 0 ? 1u : 0u);
        }
        tc05_commit(&s_full);
        tc05_commit(&k_empty[stage]);                // the keys of this tile are not needed again
      };
      bool ok = ntiles > 0 && mbar_wait(&k_full[0], 0);
      if (ok) { tc05_fence_after_sync(); issue_s(0); }
      for (int t = 0; t < ntiles && ok; ++t) {
        const int stage = t % STAGES;
        if (t + 1 < ntiles) {              // the next S runs while the rows of this one are being worked on
          ok = mbar_wait(&k_full[(t + 1) % STAGES], (unsigned)(((t + 1) / STAGES) & 1)) && mbar_wait(&s_free, (unsigned)(t & 1));
          if (!ok) break;
          tc05_fence_after_sync();
          issue_s(t + 1);
        }
        ok = mbar_wait(&p_full, (unsigned)(t & 1)) && mbar_wait(&v_full[stage], (unsigned)((t / STAGES) & 1));
        if (!ok) break;
        tc05_fence_after_sync();
        // O[128, HS] (+)= P[128, 128 keys] V_t[128 keys, HS]: 8 steps of 16 keys; V rows are keys (MN-major B)
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const unsigned long long pd = umma_desc_sw128(Ps + (size_t)(kk >> 2) * (BM * 64), 16, 1024) + 2 * (kk & 3);
          const unsigned long long vd = umma_desc_sw128(Vs + (size_t)stage * TILE, BN * 128, 1024) + 128 * kk;
          tc05_mma_bf16(tmem + TM_T, pd, vd, idesc_t, (t | kk) != 0 ? 1u : 0u);
        }
        tc05_commit(&t_full);
        tc05_commit(&v_empty[stage]);
      }
      if (!ok && ntiles > 0) { set_status(p.status, SI_WAIT_LIMIT); s_abort = 1; }
    }
  } else {
    // ---- two threads per row: column half `wg` of every tile
    constexpr int HALF = BN / 2, OH = HS / 2;        // keys of S and columns of O per thread
    const int wg = warp >> 2;
    const int r = threadIdx.x & (BM - 1);            // tile row = tensor-memory lane
    const int tok = r / p.G, hh = r - tok * p.G;
    const int pos = tok < item.ntok ? item.pos0 + tok : -1;
    const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
    float m = -INFINITY, l = 0.f;                    // base of the exponentials (log2 domain), this half's sum
    bool alive = true;
    // Every warp runs all iterations and meets the others at the named barrier in each of them, also
    // after a wait has run out (`alive` false: it then skips the work), so nobody is left waiting there.
    for (int t = 0; t < ntiles; ++t) {
      const int j0 = kv_begin + t * BN + wg * HALF;
      if (alive) alive = __all_sync(0xffffffffu, mbar_wait(&s_full, (unsigned)(t & 1)));
      float s[HALF];
      float mx = -INFINITY;
      if (alive) {
        tc05_fence_after_sync();
#pragma unroll
        for (int c = 0; c < HALF / 32; ++c) tmem_ld_32x32_issue(tmem + lane_base + TM_S + wg * HALF + c * 32, s + c * 32);
        tmem_ld_wait();
        tc05_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free);         // S may be overwritten by the next tile's product
        const bool all_visible = j0 + HALF - 1 <= pos && (p.window <= 0 || j0 > pos - p.window);
        if (all_visible) {                           // most tiles lie wholly before the row's position
#pragma unroll
          for (int i = 0; i < HALF; ++i) { s[i] *= p.scale_log2; mx = fmaxf(mx, s[i]); }
        } else {
#pragma unroll
          for (int i = 0; i < HALF; ++i) {
            const int j = j0 + i;
            const bool vis = j <= pos && (p.window <= 0 || j > pos - p.window);
            s[i] = vis ? s[i] * p.scale_log2 : -INFINITY;
            mx = fmaxf(mx, s[i]);
          }
        }
      }
      xmax[t & 1][wg][r] = mx;
      asm volatile("bar.sync 1, 256;\n" ::: "memory");
      if (!alive) continue;
      mx = fmaxf(mx, xmax[t & 1][wg ^ 1][r]);
      // raise the base only when the maximum has outgrown it by 2^8; then O and l are rescaled
      float factor = 1.f;
      const bool raise = mx > m + 8.f;
      if (raise) { factor = exp2f(m - mx); m = mx; }
      const float base = m == -INFINITY ? 0.f : m;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < HALF; ++i) { s[i] = fast_exp2(s[i] - base); sum += s[i]; }
      l = l * factor + sum;
      // P and O belong to the previous product until it has completed
      if (t > 0) {
        alive = __all_sync(0xffffffffu, mbar_wait(&t_full, (unsigned)((t - 1) & 1)));
        if (!alive) continue;
        tc05_fence_after_sync();
        if (__any_sync(0xffffffffu, raise)) {
#pragma unroll 1
          for (int c = 0; c < OH / 32; ++c) {
            float v[32];
            tmem_ld_32x32(tmem + lane_base + TM_T + wg * OH + c * 32, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= factor;
            tmem_st_32x32(tmem + lane_base + TM_T + wg * OH + c * 32, v);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < HALF / 8; ++c) {
        uint4 raw;
        raw.x = pack_bf16(s[8 * c], s[8 * c + 1]);
        raw.y = pack_bf16(s[8 * c + 2], s[8 * c + 3]);
        raw.z = pack_bf16(s[8 * c + 4], s[8 * c + 5]);
        raw.w = pack_bf16(s[8 * c + 6], s[8 * c + 7]);
        *reinterpret_cast<uint4*>(half_ptr<BM>(Ps, r, wg * (HALF / 8) + c)) = raw;
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      tc05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
    }
    if (alive && ntiles > 0) {
      const bool ok = mbar_wait(&t_full, (unsigned)((ntiles - 1) & 1));
      if (!__all_sync(0xffffffffu, ok)) alive = false;
    }
    // the two halves of a row add their sums (a failed wait anywhere is seen by all through s_abort)
    if (!alive && lane == 0) { set_status(p.status, SI_WAIT_LIMIT); s_abort = 1; }
    xsum[wg][r] = l;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    if (!s_abort) {
      tc05_fence_after_sync();
      const float lt = l + xsum[wg ^ 1][r];
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      bf16* dst = p.out + (size_t)(item.row0 + tok) * p.out_stride + (size_t)(g * p.G + hh) * p.hs + wg * OH;
#pragma unroll 1
      for (int c = 0; c < OH / 32; ++c) {
        float v[32];
        tmem_ld_32x32(tmem + lane_base + TM_T + wg * OH + c * 32, v);
        if (tok < item.ntok) {
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            uint4 raw;
            raw.x = pack_bf16(v[8 * q8] * inv, v[8 * q8 + 1] * inv);
            raw.y = pack_bf16(v[8 * q8 + 2] * inv, v[8 * q8 + 3] * inv);
            raw.z = pack_bf16(v[8 * q8 + 4] * inv, v[8 * q8 + 5] * inv);
            raw.w = pack_bf16(v[8 * q8 + 6] * inv, v[8 * q8 + 7] * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + q8 * 8) = raw;
          }
        }
      }
    }
  }
  tc05_fence_before_sync();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, TM_COLS);
}

// ---- host side --------------------------------------------------------------------------------
// 1 when this kernel takes the layout.
SI_EXPORT int si_attn_portion_tc05_ok(int H, int KV, int hs, int page_size) {
  if (KV <= 0 || H % KV || H / KV > 128) return 0;
  if (hs != 64 && hs != 128) return 0;
  if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return 0;
  return si_encode_fn() != nullptr;
}

// Tokens of one item: floor(128 / G).
SI_EXPORT int si_attn_portion_tc05_tokens(int H, int KV) { return 128 / (H / KV); }

template <int NH>
static int launch(const AttnParams& p, const CUtensorMap& km, const CUtensorMap& vm, int num_items, int log2_page,
                  cudaStream_t stream) {
  constexpr int HS = NH * 64;
  const size_t smem = (size_t)(128 * HS + 128 * 128 + 2 * 2 * NH * 128 * 64) * sizeof(bf16) + 1024;
  auto k = attn_portion_tc05_kernel<NH>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  k<<<dim3(num_items, p.KV), 320, smem, stream>>>(p, km, vm, log2_page);
  return si_last_error();
}

// Same contract as si_attn_portion (attention_mma.cu) with the tensor maps of the layer's K and V cache
// (made by si_attn_encode_cache_map of attention_tma.cu); items hold at most si_attn_portion_tc05_tokens().
SI_EXPORT int si_attn_portion_tc05(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                   const void* kmap, const void* vmap, const int* block_table, int table_width,
                                   const void* items, int num_items, void* out, long long out_stride, int num_pages,
                                   int page_size, int num_seqs, int H, int KV, int hs, float scale, int window,
                                   int* status, cudaStream_t stream) {
  if (num_items <= 0) return 0;
  if (!si_attn_portion_tc05_ok(H, KV, hs, page_size) || !kmap || !vmap) return -2;
  if ((q_stride % 8) || (out_stride % 8) || ((uintptr_t)q % 16) || ((uintptr_t)out % 16)) return -2;
  AttnParams p;
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
  int log2_page = 0;
  while ((1 << log2_page) < page_size) ++log2_page;
  const CUtensorMap& km = *(const CUtensorMap*)kmap;
  const CUtensorMap& vm = *(const CUtensorMap*)vmap;
  return hs == 64 ? launch<1>(p, km, vm, num_items, log2_page, stream) : launch<2>(p, km, vm, num_items, log2_page, stream);
}
