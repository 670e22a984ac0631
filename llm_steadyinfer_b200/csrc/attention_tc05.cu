// Attention for prompt portions on the 5th-generation tensor cores (tcgen05), bf16, over the
// paged cache. One block handles one work item (a run of consecutive query tokens of a sequence)
// for one KV head as TWO query tiles of 128 rows each (row r of a tile = token r / G of the tile,
// head r % G; a tile holds floor(128 / G) tokens), against key tiles of 128. The two query tiles
// share every K and V tile and take turns: while the rows of one are in the softmax, the tensor
// cores work for the other.
//
//   warp 8 (producer)  looks up the pages of a key tile and issues its K and V boxes by TMA
//                      (128-byte swizzle) into one of two stages;
//   warp 9 (issuer)    per query tile: S = Q K^T with tcgen05.mma into tensor memory (Q, K K-major) and,
//                      once the probabilities stand in tensor memory, O += P V with P as the
//                      tensor-memory A operand and V the MN-major B operand, as it lies in the cache.
//                      Its order of issue, P V and the next S of tile 0, then of tile 1, keeps the two
//                      tiles in opposite phases: one in the softmax while the tensor cores serve the other;
//   warps 0-3 / 4-7    one thread per row of query tile 0 / 1: reads the row of S (tcgen05.ld), takes its
//                      maximum, computes exp2 of the scaled scores in fp32 against a base that is raised
//                      only when the maximum has grown by more than 2^8 (then the row of O in tensor
//                      memory is rescaled first), and writes the bf16 probabilities over the first
//                      columns of S (tcgen05.st); at the end it reads O and divides by the row sum.
//
// The tensor cores run one thread's instructions in the order of issue, which is what keeps this
// simple: S of the next key tile is issued behind P V of the current one, so it overwrites P only
// after P has been read, and when S is complete so is every earlier product into O.
//
// The reference computes prompt attention row by row with its scalar split kernel
// (src/source/op/kernels/cuda/paged_kernels.cu:96-206). Conditions here: head_dim 64 or 128, page size
// a power of two from 8 to 64, G <= 128; other layouts use the mma.sync kernel. Every mbarrier wait
// is bounded; when one runs out the block sets SI_WAIT_LIMIT and leaves without storing.
#include "attention_common.cuh"
#include "tma_common.cuh"
#include <limits.h>

// Packed fp32 arithmetic of sm_100 in the softmax (two scores an instruction) and three-input maxima.
#ifndef SI_ATTN_PACKED
#define SI_ATTN_PACKED 1
#endif
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
  unsigned long long v;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
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
  constexpr int TM_S = 0, TM_O = 2 * BN;             // tensor-memory columns: S of tile q at TM_S + q*BN, O at TM_O + q*HS
  constexpr int TM_COLS = 512;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
  __shared__ __align__(8) uint64_t s_full[2], p_full[2], o_full[2];   // per query tile
  __shared__ unsigned tmem_slot;
  __shared__ int s_abort;
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);     // [2 tiles][NH][128][64]
  bf16* Ks = Qs + 2 * BM * HS;                       // [STAGES][TILE]
  bf16* Vs = Ks + STAGES * TILE;

  // Items of a prompt come in order of position, so the last ones have the most keys: start with those,
  // for all KV heads alike (blocks are handed out with x running fastest, and x is the KV head).
  const AttnItem item = p.items[gridDim.y - 1 - blockIdx.y];
  if (item.ntok <= 0) return;
  const int g = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (item.seq < 0 || item.seq >= p.num_seqs) {
    if (threadIdx.x == 0) set_status(p.status, SI_BAD_SEQ);
    return;
  }
  const int* table = p.block_table + (size_t)item.seq * p.table_width;
  const int tile_tokens = BM / p.G;                  // tokens of one query tile
  const bool two = item.ntok > tile_tokens;          // the second query tile has rows
  const int kv_end = item.pos0 + item.ntok;
  const int kv_lo = window_first_key(item.pos0, p.window);
  const int kv_begin = kv_lo / BN * BN;
  const int ntiles = (kv_end - kv_begin + BN - 1) / BN;
  const int page_rows = 1 << log2_page;
  const int pages_per_tile = BN >> log2_page;

  pdl_trigger();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      mbar_init(&s_full[q], 1);
      mbar_init(&p_full[q], 4);                      // one arrival per warp of the tile's rows
      mbar_init(&o_full[q], 1);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 9) tmem_alloc(&tmem_slot, TM_COLS);
  // rows that no copy fills must hold finite numbers (they meet zero probabilities): those behind the
  // last key in the last tile, and pages wholly before the window in the first
  auto clear_stage = [&](int stage) {
    uint4* kz = reinterpret_cast<uint4*>(Ks + (size_t)stage * TILE);
    uint4* vz = reinterpret_cast<uint4*>(Vs + (size_t)stage * TILE);
    for (int i = threadIdx.x; i < TILE / 8; i += blockDim.x) { kz[i] = make_uint4(0, 0, 0, 0); vz[i] = make_uint4(0, 0, 0, 0); }
  };
  if ((kv_end - kv_begin) % BN != 0) clear_stage((ntiles - 1) % STAGES);
  if (kv_begin + page_rows <= kv_lo) clear_stage(0);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  tc05_fence_before_sync();
  __syncthreads();                                   // barriers, tensor memory and the zeroed rows stand
  // launched as a programmatic dependent, all of the above ran while the kernel before this one (which wrote the
  // queries and the newest keys and values) was ending; the items and the block table were copied in earlier
  pdl_wait();
  tc05_fence_after_sync();
  const unsigned tmem = tmem_slot;
  if (warp != 8) {
    // Query rows, while the producer already fetches the first keys: row r of tile q is token
    // q * tile_tokens + r / G, head g*G + r % G. All loads of a thread are issued before its stores.
    constexpr int NT = 288, PER = (2 * BM * (HS / 8) + NT - 1) / NT;
    const int tid = warp == 9 ? 256 + lane : threadIdx.x;
    const int rows = two ? 2 * BM : BM;              // the second tile is not read when it has no token
    uint4 v[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int id = tid + i * NT;
      const int row = id / (HS / 8), c = id % (HS / 8);
      const int q = row / BM, r = row % BM;
      const int tl = r / p.G, hh = r - tl * p.G;
      const int tok = q * tile_tokens + tl;
      v[i] = make_uint4(0, 0, 0, 0);
      if (row < rows && tl < tile_tokens && tok < item.ntok)
        v[i] = *reinterpret_cast<const uint4*>(p.q + (size_t)(item.row0 + tok) * p.q_stride + (size_t)(g * p.G + hh) * p.hs + c * 8);
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int id = tid + i * NT;
      const int row = id / (HS / 8), c = id % (HS / 8);
      if (row < rows) *reinterpret_cast<uint4*>(half_ptr<BM>(Qs + (size_t)(row / BM) * BM * HS, row % BM, c)) = v[i];
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    asm volatile("bar.sync 1, 288;\n" ::: "memory");   // warps 0-7 and 9
  }

  if (warp == 8) {
    // ---- producer: box b = (page, half, K or V) of each tile, boxes spread over the lanes. K and V
    // have barriers of their own: a K stage is free as soon as both S have been computed from it, long
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
        // pages past the last key, or wholly before the window, are not fetched
        if (b < boxes && j + pg * page_rows < kv_end && j + (pg + 1) * page_rows > kv_lo) {
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
      if (t >= STAGES) ok = mbar_wait_warp(&k_empty[stage], (unsigned)(((t / STAGES) - 1) & 1));
      if (!ok) {
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
      if (t >= STAGES) ok = mbar_wait_warp(&v_empty[stage], (unsigned)(((t / STAGES) - 1) & 1));
      if (!ok) {
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
    // ---- issuer: S_0(0) S_1(0) | P V_0(0) S_0(1) | P V_1(0) S_1(1) | P V_0(1) S_0(2) | ...
    // The whole warp runs this code and one elected lane issues: what an instruction needs (descriptors,
    // addresses) is then uniform over the warp. The descriptors are made once and only their address
    // fields (units of 16 bytes) advance. An instruction is accepted only as fast as the tensor cores
    // run, so whatever else this warp does between two of them leaves the tensor cores idle.
    constexpr unsigned idesc_s = umma_idesc_bf16(BM, BN, false);
    constexpr unsigned idesc_o = umma_idesc_bf16(BM, HS, true);
    constexpr unsigned U_TILE = TILE * 2 / 16, U_QTILE = BM * HS * 2 / 16, U_HALF = BN * 64 * 2 / 16;
    const int nq = two ? 2 : 1;
    const unsigned long long qd0 = umma_desc_sw128(Qs, 16, 1024);
    const unsigned long long kd0 = umma_desc_sw128(Ks, 16, 1024);
    const unsigned long long vd0 = umma_desc_sw128(Vs, BN * 128, 1024);
    auto issue_s = [&](int q, int t) {  // S_q[128, 128] = Q_q[128, HS] K_t[128 keys, HS]^T: 4 steps per 64-column half
      const unsigned long long qd = qd0 + (unsigned)q * U_QTILE;
      const unsigned long long kd = kd0 + (unsigned)(t % STAGES) * U_TILE;
      const unsigned sd = tmem + TM_S + q * BN;
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < HS / 16; ++kk)
          tc05_mma_bf16(sd, qd + ((kk >> 2) * U_HALF + 2 * (kk & 3)), kd + ((kk >> 2) * U_HALF + 2 * (kk & 3)), idesc_s, kk != 0 ? 1u : 0u);
        tc05_commit(&s_full[q]);
        if (q == nq - 1) tc05_commit(&k_empty[t % STAGES]);      // the keys of this tile are not needed again
      }
      __syncwarp();
    };
    bool ok = ntiles > 0 && mbar_wait_warp(&k_full[0], 0);
    if (ok) {
      tc05_fence_after_sync();
      for (int q = 0; q < nq; ++q) issue_s(q, 0);
    }
    for (int t = 0; t < ntiles && ok; ++t) {
      const int stage = t % STAGES;
      const bool more = t + 1 < ntiles;
      ok = mbar_wait_warp(&v_full[stage], (unsigned)((t / STAGES) & 1));
      for (int q = 0; q < nq && ok; ++q) {
        ok = mbar_wait_warp(&p_full[q], (unsigned)(t & 1));
        if (!ok) break;
        tc05_fence_after_sync();
        // O_q[128, HS] (+)= P_q[128, 128 keys] V_t[128 keys, HS]: 8 steps of 16 keys; P lies packed in the first
        // 64 columns of S_q, V rows are keys (MN-major B)
        const unsigned long long vd = vd0 + (unsigned)stage * U_TILE;
        const unsigned sd = tmem + TM_S + q * BN, od = tmem + TM_O + q * HS;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            tc05_mma_bf16_tmem_a(od, sd + 8 * kk, vd + 128 * kk, idesc_o, (t | kk) != 0 ? 1u : 0u);
          if (!more) tc05_commit(&o_full[q]);
          if (q == nq - 1) tc05_commit(&v_empty[stage]);
        }
        __syncwarp();
        if (more) {                        // behind P V in the order of issue: S overwrites P only after it was read
          if (q == 0) ok = mbar_wait_warp(&k_full[(t + 1) % STAGES], (unsigned)(((t + 1) / STAGES) & 1));
          if (!ok) break;
          tc05_fence_after_sync();
          issue_s(q, t + 1);
        }
      }
    }
    if (!ok && ntiles > 0 && lane == 0) { set_status(p.status, SI_WAIT_LIMIT); s_abort = 1; }
  } else if (warp < 4 || two) {
    // ---- one thread per row of query tile q
    const int q = warp >> 2;
    const int r = threadIdx.x & (BM - 1);            // tile row = tensor-memory lane
    const int tl = r / p.G, hh = r - tl * p.G;
    const int tok = q * tile_tokens + tl;
    const bool valid = tl < tile_tokens && tok < item.ntok;
    const int pos = valid ? item.pos0 + tok : -1;
    const int lo = p.window > 0 ? pos - p.window + 1 : INT_MIN;     // visible keys: lo <= j <= pos
    const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
    const unsigned ts = tmem + lane_base + TM_S + q * BN, to = tmem + lane_base + TM_O + q * HS;
    float m = -INFINITY, l = 0.f;                    // base of the exponentials (log2 domain), the row's sum
    bool alive = true;
    for (int t = 0; t < ntiles; ++t) {
      const int j0 = kv_begin + t * BN;
      alive = mbar_wait_warp(&s_full[q], (unsigned)(t & 1));
      if (!alive) break;
      tc05_fence_after_sync();
      float s[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tmem_ld_32x32_issue(ts + 32 * c, s + 32 * c);
      tmem_ld_wait();
      // most tiles lie wholly inside every row's visible range: then nothing is masked
      if (__any_sync(0xffffffffu, !(j0 >= lo && j0 + BN - 1 <= pos))) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int j = j0 + i;
          if (j < lo || j > pos) s[i] = -INFINITY;
        }
      }
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#if SI_ATTN_PACKED
#pragma unroll
      for (int i = 0; i < BN; i += 8) {                    // three-input maxima: half the instructions
        m4[0] = max3(m4[0], s[i], s[i + 1]); m4[1] = max3(m4[1], s[i + 2], s[i + 3]);
        m4[2] = max3(m4[2], s[i + 4], s[i + 5]); m4[3] = max3(m4[3], s[i + 6], s[i + 7]);
      }
#else
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        m4[0] = fmaxf(m4[0], s[i]); m4[1] = fmaxf(m4[1], s[i + 1]);
        m4[2] = fmaxf(m4[2], s[i + 2]); m4[3] = fmaxf(m4[3], s[i + 3]);
      }
#endif
      // the scale is positive, so the maximum may be taken before it
      const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;
      // raise the base only when the maximum has outgrown it by 2^8; then O and l are rescaled. S being
      // complete, so is every earlier product into O.
      float factor = 1.f;
      const bool raise = mx > m + 8.f;
      if (raise) { factor = fast_exp2(m - mx); m = mx; }   // exp2(-inf) = 0 on the first keys
      if (t > 0 && __any_sync(0xffffffffu, raise)) {
#pragma unroll 1
        for (int c = 0; c < HS / 32; ++c) {
          float v[32];
          tmem_ld_32x32(to + c * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= factor;
          tmem_st_32x32(to + c * 32, v);
        }
      }
      const float base = m == -INFINITY ? 0.f : m;
#if SI_ATTN_PACKED
      // scale, subtraction of the base and the row's sum two scores at a time (fma.rn.f32x2, add.rn.f32x2: the
      // same roundings as the single instructions, half as many of them)
      const unsigned long long sc2 = pack_f32x2(p.scale_log2, p.scale_log2), nb2 = pack_f32x2(-base, -base);
      unsigned long long sum2[2] = {0ull, 0ull};
#pragma unroll
      for (int b = 0; b < BN / 64; ++b) {
        unsigned pk[32];
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          float e[4];
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            float x0, x1;
            unpack_f32x2(fma_f32x2(pack_f32x2(s[64 * b + i + 2 * w], s[64 * b + i + 2 * w + 1]), sc2, nb2), x0, x1);
            e[2 * w] = fast_exp2(x0);                      // exp2(-inf) = 0 for masked keys
            e[2 * w + 1] = fast_exp2(x1);
            sum2[w] = add_f32x2(sum2[w], pack_f32x2(e[2 * w], e[2 * w + 1]));
          }
          pk[i / 2] = pack_bf16(e[0], e[1]);
          pk[i / 2 + 1] = pack_bf16(e[2], e[3]);
        }
        // the probabilities of keys 64b .. 64b+63 go over columns 32b .. 32b+31 of S, which is in registers
        tmem_st_32x32_issue(ts + 32 * b, pk);
      }
      float s4[4];
      unpack_f32x2(sum2[0], s4[0], s4[1]);
      unpack_f32x2(sum2[1], s4[2], s4[3]);
      l = l * factor + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
#else
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int b = 0; b < BN / 64; ++b) {
        unsigned pk[32];
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float e = fast_exp2(fmaf(s[64 * b + i + w], p.scale_log2, -base));    // exp2(-inf) = 0 for masked keys
            s[64 * b + i + w] = e;
            s4[w] += e;
          }
          pk[i / 2] = pack_bf16(s[64 * b + i], s[64 * b + i + 1]);
          pk[i / 2 + 1] = pack_bf16(s[64 * b + i + 2], s[64 * b + i + 3]);
        }
        // the probabilities of keys 64b .. 64b+63 go over columns 32b .. 32b+31 of S, which is in registers
        tmem_st_32x32_issue(ts + 32 * b, pk);
      }
      l = l * factor + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
#endif
      tmem_st_wait();
      tc05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[q]);
    }
    if (alive && ntiles > 0) alive = mbar_wait_warp(&o_full[q], 0);
    if (!alive && lane == 0) { set_status(p.status, SI_WAIT_LIMIT); s_abort = 1; }
    if (alive) {
      tc05_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      bf16* dst = p.out + (size_t)(item.row0 + tok) * p.out_stride + (size_t)(g * p.G + hh) * p.hs;
#pragma unroll
      for (int c = 0; c < HS / 64; ++c) {
        float v[64];
        tmem_ld_32x32_issue(to + c * 64, v);
        tmem_ld_32x32_issue(to + c * 64 + 32, v + 32);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int q8 = 0; q8 < 8; ++q8) {
            uint4 raw;
            raw.x = pack_bf16(v[8 * q8] * inv, v[8 * q8 + 1] * inv);
            raw.y = pack_bf16(v[8 * q8 + 2] * inv, v[8 * q8 + 3] * inv);
            raw.z = pack_bf16(v[8 * q8 + 4] * inv, v[8 * q8 + 5] * inv);
            raw.w = pack_bf16(v[8 * q8 + 6] * inv, v[8 * q8 + 7] * inv);
            *reinterpret_cast<uint4*>(dst + c * 64 + q8 * 8) = raw;
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

// Tokens of one item: two query tiles of floor(128 / G) each.
SI_EXPORT int si_attn_portion_tc05_tokens(int H, int KV) { return 2 * (128 / (H / KV)); }

template <int NH>
static int launch(const AttnParams& p, const CUtensorMap& km, const CUtensorMap& vm, int num_items, int log2_page,
                  cudaStream_t stream) {
  constexpr int HS = NH * 64;
  // Q of both query tiles, two stages of K and of V. The block takes all of tensor memory, so a second
  // block on the same SM could only wait for it: ask for more than half of the shared memory.
  size_t smem = (size_t)(2 * 128 * HS + 2 * 2 * NH * 128 * 64) * sizeof(bf16) + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;
  auto k = attn_portion_tc05_kernel<NH>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  si_launch(k, dim3(p.KV, num_items), dim3(320), smem, stream, p, km, vm, log2_page);
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
  if (num_items > 65535) return -2;                  // the grid's second dimension
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
