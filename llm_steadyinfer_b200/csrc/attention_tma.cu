// Decode attention over the paged cache with the K/V tiles brought in by TMA.
//
// Same arithmetic as `attn_decode_kernel` (attention_mma.cu): 16*MT rows (tokens x query heads
// of one KV head) shared by four warps, each warp taking 16 of the 64 keys of a tile, bf16
// mma.sync with fp32 accumulation and fp32 online softmax, optional split of the key range over
// blocks with the last block merging. What differs is how tiles reach shared memory: one page of
// one KV head is a contiguous [page_size, head_dim] slab of the cache, so a 64-key tile is
// 64 / page_size boxes per 64-column half of K and of V. One elected thread issues them as
// `cp.async.bulk.tensor.2d` copies with the 128-byte swizzle (which is the XOR layout ldmatrix
// wants). A fifth warp is the producer: its lanes look up the pages and issue the boxes of a tile,
// one box a lane, as soon as the four consumer warps have released the stage (`empty` mbarrier);
// a `full` mbarrier per stage counts the bytes in. The consumer warps spend no instructions on
// addresses, which the cp.async version pays about 400 of per thread and tile, and never meet
// at a block-wide barrier inside the loop.
//
// Conditions: head_dim 64 or 128, page_size a power of two from 8 to 64, at most 32 rows per
// item. Everything else stays with the cp.async kernel. Every wait on an mbarrier is bounded:
// when it runs out the block reports SI_WAIT_LIMIT in the status word and leaves.
#include "attention_common.cuh"
#include "tma_common.cuh"

// Tile of NROWS rows stored as 64-column halves; inside a half, row r holds its eight 16-byte
// chunks at positions chunk ^ (r % 8): the layout the 128-byte TMA swizzle writes.
template <int NROWS>
__device__ __forceinline__ bf16* half_tile_ptr(bf16* base, int row, int chunk) {
  return base + (size_t)(chunk >> 3) * (NROWS * 64) + (size_t)row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}

// m8n8 transpose of 16-bit elements across the warp: lane (g, t) gives row g, columns 2t and 2t+1 and gets
// row g, columns 2t and 2t+1 of the transposed matrix.
__device__ __forceinline__ unsigned movmatrix_trans(unsigned v) {
  unsigned r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(v));
  return r;
}

// SWAP (items of at most 8 rows, the usual decode step): the products are taken the other way round,
// S^T = K Q^T and O^T = V^T P^T, so that the 16 rows of the tensor-core instruction are keys (or
// head-dim elements) and its 8 columns the query rows. With the rows as the 16 of the instruction
// three quarters of every product and of the softmax arithmetic are spent on rows that do not exist;
// this way a tile costs half the instructions, and the consumer warps, one per scheduler, are bound
// by their instruction stream.
template <int NH, int MT, int STAGES, bool SWAP>
__global__ void __launch_bounds__(160)
attn_decode_tma_kernel(const AttnParams p, const __grid_constant__ CUtensorMap kmap,
                       const __grid_constant__ CUtensorMap vmap, int log2_page, const int4* __restrict__ work, int trigger) {
  constexpr int NWARPS = 4, THREADS = 128, BLOCK_N = 64, ROWS = 16 * MT, HS_PAD = NH * 64;   // consumer warps/threads
  constexpr int KT = HS_PAD / 16, DT = HS_PAD / 8;
  constexpr int TILE = NH * BLOCK_N * 64;             // elements of one K (or V) tile
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ int s_last;
  __shared__ int s_abort;
  unsigned char* smem_raw = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  bf16* Ks = reinterpret_cast<bf16*>(smem_raw);     // [STAGES][TILE]
  bf16* Vs = Ks + STAGES * TILE;
  bf16* Qs = Vs + STAGES * TILE;                     // [NH][ROWS][64]

  if (trigger) pdl_trigger();
  // Until its pdl_wait() below no thread reads what the kernel before this one writes (the queries and the
  // newest keys and values): the work list, the items and the block table were copied in before it began.
  // Which share of which item: with a work list, entry blockIdx.x = (item, split, splits of the item, first
  // partial-result slot of the item), so that long sequences are cut into more shares than short ones;
  // without one, item blockIdx.x and split blockIdx.z of p.nsplit.
  int item_idx = blockIdx.x, split = blockIdx.z, nsplit = p.nsplit, slot0 = blockIdx.x * p.nsplit;
  if (work) {
    const int4 w = work[blockIdx.x];
    if (w.x < 0) return;                           // entries behind the step's last one
    item_idx = w.x; split = w.y; nsplit = w.z; slot0 = w.w;
  }
  const AttnItem item = p.items[item_idx];
  if (item.ntok <= 0) return;
  const int g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (item.seq < 0 || item.seq >= p.num_seqs) {
    if (threadIdx.x == 0) set_status(p.status, SI_BAD_SEQ);
    return;
  }
  const int* table = p.block_table + (size_t)item.seq * p.table_width;
  const int kv_end_all = item.pos0 + item.ntok;
  const int kv_lo = window_first_key(item.pos0, p.window);
  const int kv_begin_all = kv_lo / BLOCK_N * BLOCK_N;
  const int tiles_all = (kv_end_all - kv_begin_all + BLOCK_N - 1) / BLOCK_N;
  const int tiles_per = (tiles_all + nsplit - 1) / nsplit;
  const int t_begin = split * tiles_per;
  const int t_end = min(tiles_all, t_begin + tiles_per);
  const int ntiles = max(0, t_end - t_begin);
  const int kv_begin = kv_begin_all + t_begin * BLOCK_N;
  const int kv_end = min(kv_end_all, kv_begin_all + t_end * BLOCK_N);
  const int page_rows = 1 << log2_page;
  const int pages_per_tile = BLOCK_N >> log2_page;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], NWARPS); }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // Rows that no copy fills must hold finite numbers (they meet zero probabilities): clear the stage
  // the last tile lands in if keys end inside it, and the first one if pages of it lie wholly before
  // the window.
  auto clear_stage = [&](int stage) {
    uint4* kz = reinterpret_cast<uint4*>(Ks + (size_t)stage * TILE);
    uint4* vz = reinterpret_cast<uint4*>(Vs + (size_t)stage * TILE);
    for (int i = threadIdx.x; i < TILE / 8; i += blockDim.x) { kz[i] = make_uint4(0, 0, 0, 0); vz[i] = make_uint4(0, 0, 0, 0); }
  };
  if (ntiles > 0 && (kv_end - kv_begin) % BLOCK_N != 0) clear_stage((ntiles - 1) % STAGES);
  if (ntiles > 0 && kv_begin + page_rows <= kv_lo) clear_stage(0);
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  __syncthreads();                              // the barriers stand, the cleared rows are there for the copies
  if (warp < NWARPS) {
    pdl_wait();
    // query rows: tile row r is token r / G, head g*G + r % G
    for (int id = threadIdx.x; id < ROWS * (HS_PAD / 8); id += THREADS) {
      const int row = id / (HS_PAD / 8), c = id % (HS_PAD / 8);
      const int tok = row / p.G, hh = row - tok * p.G;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (tok < item.ntok && c * 8 < p.hs)
        v = *reinterpret_cast<const uint4*>(p.q + (size_t)(item.row0 + tok) * p.q_stride + (size_t)(g * p.G + hh) * p.hs + c * 8);
      *reinterpret_cast<uint4*>(half_tile_ptr<ROWS>(Qs, row, c)) = v;
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
  }

  if (warp == NWARPS) {
    // ---- producer warp: lane l fetches box (page l / (2 NH), half (l / 2) % NH, K or V) of each tile
    const int boxes = pages_per_tile * NH * 2;
    const int pg = lane / (2 * NH), h = (lane >> 1) % NH, is_v = lane & 1;
    // The page numbers are read three tiles ahead: a lookup in the loop would put the latency of a load
    // from global memory into every tile's turn.
    constexpr int NOT_NEEDED = -2;
    auto lookup = [&](int t) {
      const int j = kv_begin + t * BLOCK_N;
      // pages past the last key, or wholly before the window, are not fetched
      if (t >= ntiles || lane >= boxes || j + pg * page_rows >= kv_end || j + (pg + 1) * page_rows <= kv_lo) return NOT_NEEDED;
      const int slot = (j >> log2_page) + pg;
      return slot < p.table_width ? __ldg(table + slot) : -1;
    };
    int ahead0 = lookup(0), ahead1 = lookup(1), ahead2 = lookup(2);
    // Tiles that end before the item's first position hold nothing that the kernel before this one writes
    // (it stores the keys and values of the step's own tokens): their copies start before this kernel waits.
    bool waited = false;
    for (int t = 0; t < ntiles; ++t) {
      if (!waited && kv_begin + (t + 1) * BLOCK_N > item.pos0) { pdl_wait(); waited = true; }
      const int stage = t % STAGES;
      int page = ahead0;
      ahead0 = ahead1; ahead1 = ahead2; ahead2 = lookup(t + 3);
      if (page != NOT_NEEDED && (page < 0 || page >= p.num_pages)) { set_status(p.status, SI_BAD_PAGE); page = -1; }
      const unsigned have = __ballot_sync(0xffffffffu, page >= 0);
      bool ok = true;
      if (t >= STAGES) ok = mbar_wait(&empty_bar[stage], (unsigned)(((t / STAGES) - 1) & 1));
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) { set_status(p.status, SI_WAIT_LIMIT); s_abort = 1; }
        break;
      }
      if (lane == 0) mbar_expect_tx(&full_bar[stage], (unsigned)(__popc(have) * page_rows * 128));
      __syncwarp();
      if (page >= 0) {
        const int row = (page * p.KV + g) << log2_page;
        const size_t off = (size_t)stage * TILE + (size_t)h * (BLOCK_N * 64) + (size_t)(pg * page_rows) * 64;
        tma_load_2d((is_v ? Vs : Ks) + off, is_v ? &vmap : &kmap, &full_bar[stage], h * 64, row);
      }
    }
  }

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

  // The query fragments do not change from tile to tile: they are read from shared memory once.
  unsigned qf[MT][KT][4];
  int pos_min = 0x7fffffff, pos_max = -1;            // over the rows of this lane's fragments
  if constexpr (SWAP) {
    // lane (g, t): B fragment of Q^T, row g, head-dim elements 16kk + 2t, +1 and 16kk + 8 + 2t, +1;
    // the lane's elements of S^T belong to rows 2t and 2t + 1
    static_assert(!SWAP || MT == 1, "the swapped products take one 8-row tile");
    if (warp < NWARPS) {
#pragma unroll
      for (int kk = 0; kk < KT; ++kk) {
        qf[0][kk][0] = *reinterpret_cast<const unsigned*>(half_tile_ptr<ROWS>(Qs, lane >> 2, kk * 2) + 2 * (lane & 3));
        qf[0][kk][1] = *reinterpret_cast<const unsigned*>(half_tile_ptr<ROWS>(Qs, lane >> 2, kk * 2 + 1) + 2 * (lane & 3));
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int tok = (2 * (lane & 3) + i) / p.G;
        pos_of[0][i] = tok < item.ntok ? item.pos0 + tok : -1;
        if (pos_of[0][i] >= 0) { pos_min = min(pos_min, pos_of[0][i]); pos_max = max(pos_max, pos_of[0][i]); }
      }
    }
  } else if (warp < NWARPS) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int kk = 0; kk < KT; ++kk)
        ldsm_x4(qf[mt][kk][0], qf[mt][kk][1], qf[mt][kk][2], qf[mt][kk][3],
                half_tile_ptr<ROWS>(Qs, mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), kk * 2 + (lane >> 4)));
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2)
        if (pos_of[mt][h2] >= 0) { pos_min = min(pos_min, pos_of[mt][h2]); pos_max = max(pos_max, pos_of[mt][h2]); }   // rows without a token decide nothing
  }

  for (int t = 0; warp < NWARPS && t < ntiles; ++t) {
    const int j0 = kv_begin + t * BLOCK_N;
    const int stage = t % STAGES;
    bf16* Kt = Ks + (size_t)stage * TILE;
    bf16* Vt = Vs + (size_t)stage * TILE;
    const bool arrived = mbar_wait(&full_bar[stage], (unsigned)((t / STAGES) & 1));
    if (!__all_sync(0xffffffffu, arrived)) {
      if (lane == 0) { set_status(p.status, SI_WAIT_LIMIT); s_abort = 1; }
      break;
    }
    const int jw = j0 + warp * 16;          // this warp's 16 keys
    if (jw < kv_end) {
      // most tiles lie wholly inside every row's visible range: then nothing is masked
      const bool masked = __any_sync(0xffffffffu, jw + 15 > pos_min || (p.window > 0 && jw <= pos_max - p.window));
      if constexpr (SWAP) {
        // S^T[16 keys, 8 rows]: the lane holds keys g, g + 8 (elements 0-1, 2-3) of rows 2t, 2t + 1
        float st[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < KT; ++kk) {
          unsigned a0, a1, a2, a3;
          ldsm_x4(a0, a1, a2, a3, half_tile_ptr<BLOCK_N>(Kt, warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), kk * 2 + (lane >> 4)));
          mma_bf16(st, a0, a1, a2, a3, qf[0][kk][0], qf[0][kk][1]);
        }
        if (masked) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = jw + (lane >> 2) + 8 * (e >> 1);
            const int pos = pos_of[0][e & 1];
            if (!(j <= pos && (p.window <= 0 || j > pos - p.window))) st[e] = -INFINITY;
          }
        }
        float mx[2] = {m[0][0], m[0][1]}, corr[2], base[2];
#pragma unroll
        for (int e = 0; e < 4; ++e) { st[e] *= p.scale_log2; mx[e & 1] = fmaxf(mx[e & 1], st[e]); }
#pragma unroll
        for (int i = 0; i < 2; ++i) {                 // over the eight lanes that hold the other keys of the row
          mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 4));
          mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 8));
          mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 16));
          base[i] = mx[i] == -INFINITY ? 0.f : mx[i];
          corr[i] = fast_exp2(m[0][i] - base[i]);
          m[0][i] = mx[i];
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int e = 0; e < 4; ++e) { st[e] = fast_exp2(st[e] - base[e & 1]); sum[e & 1] += st[e]; }
        l[0][0] = l[0][0] * corr[0] + sum[0];          // this lane's keys only; the lanes are added at the end
        l[0][1] = l[0][1] * corr[1] + sum[1];
        // P^T as the B operand: transposing the 8x8 blocks turns (key g, rows 2t, 2t+1) into (row g, keys 2t, 2t+1)
        const unsigned b0 = movmatrix_trans(pack_bf16(st[0], st[1])), b1 = movmatrix_trans(pack_bf16(st[2], st[3]));
        // O^T[head dim, 8 rows] += V^T[head dim, 16 keys] P^T[16 keys, 8 rows], 16 head-dim elements a step
#pragma unroll
        for (int dm = 0; dm < HS_PAD / 16; ++dm) {
          o[0][dm][0] *= corr[0]; o[0][dm][1] *= corr[1]; o[0][dm][2] *= corr[0]; o[0][dm][3] *= corr[1];
          unsigned a0, a1, a2, a3;
          ldsm_x4_t(a0, a1, a2, a3, half_tile_ptr<BLOCK_N>(Vt, warp * 16 + (lane & 7) + 8 * (lane >> 4), dm * 2 + ((lane >> 3) & 1)));
          mma_bf16(o[0][dm], a0, a1, a2, a3, b0, b1);
        }
      } else
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KT; ++kk) {
          unsigned b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, half_tile_ptr<BLOCK_N>(Kt, warp * 16 + (lane & 7) + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
          mma_bf16(s[0], qf[mt][kk][0], qf[mt][kk][1], qf[mt][kk][2], qf[mt][kk][3], b0, b1);
          mma_bf16(s[1], qf[mt][kk][0], qf[mt][kk][1], qf[mt][kk][2], qf[mt][kk][3], b2, b3);
        }
        float mx[2] = {m[mt][0], m[mt][1]};
        if (masked) {
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j = jw + nt * 8 + (lane & 3) * 2 + (e & 1);
              const int pos = pos_of[mt][e >> 1];
              const bool vis = j <= pos && (p.window <= 0 || j > pos - p.window);
              if (!vis) s[nt][e] = -INFINITY;
            }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[nt][e] *= p.scale_log2;
            mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
          }
        float corr[2], base[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
          mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
          base[h2] = mx[h2] == -INFINITY ? 0.f : mx[h2];
          corr[h2] = fast_exp2(m[mt][h2] - base[h2]);
          m[mt][h2] = mx[h2];
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[nt][e] = fast_exp2(s[nt][e] - base[e >> 1]);
            sum[e >> 1] += s[nt][e];
          }
        l[mt][0] = l[mt][0] * corr[0] + sum[0];
        l[mt][1] = l[mt][1] * corr[1] + sum[1];
        const unsigned a0 = pack_bf16(s[0][0], s[0][1]), a1 = pack_bf16(s[0][2], s[0][3]);
        const unsigned a2 = pack_bf16(s[1][0], s[1][1]), a3 = pack_bf16(s[1][2], s[1][3]);
        {
#pragma unroll
          for (int dt = 0; dt < DT; ++dt) {
            o[mt][dt][0] *= corr[0]; o[mt][dt][1] *= corr[0]; o[mt][dt][2] *= corr[1]; o[mt][dt][3] *= corr[1];
          }
        }
#pragma unroll
        for (int dt = 0; dt < DT; dt += 2) {
          unsigned b0, b1, b2, b3;
          ldsm_x4_t(b0, b1, b2, b3, half_tile_ptr<BLOCK_N>(Vt, warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dt + (lane >> 4)));
          mma_bf16(o[mt][dt], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[mt][dt + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);      // this warp is done with the stage
  }
  __syncthreads();
  if (s_abort) return;              // a bounded wait ran out somewhere: the status word says so
  if (warp == NWARPS) return;       // the producer has nothing to merge

  // merge the warps through shared memory (all tiles have been consumed and none is in flight)
  float* fm = reinterpret_cast<float*>(smem_raw);
  float* fl = fm + NWARPS * ROWS;
  float* fo = fl + NWARPS * ROWS;
  constexpr int OS = HS_PAD + 4;
  if constexpr (SWAP) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float lv = l[0][i];
      lv += __shfl_xor_sync(0xffffffffu, lv, 4);
      lv += __shfl_xor_sync(0xffffffffu, lv, 8);
      lv += __shfl_xor_sync(0xffffffffu, lv, 16);
      const int r = 2 * (lane & 3) + i;
      if ((lane >> 2) == 0) { fm[warp * ROWS + r] = m[0][i]; fl[warp * ROWS + r] = lv; }
#pragma unroll
      for (int dm = 0; dm < HS_PAD / 16; ++dm) {
        const int d = dm * 16 + (lane >> 2);
        fo[((size_t)warp * ROWS + r) * OS + d] = o[0][dm][i];
        fo[((size_t)warp * ROWS + r) * OS + d + 8] = o[0][dm][2 + i];
      }
    }
  } else
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
  asm volatile("bar.sync 1, 128;\n" ::: "memory");
  const int rows_used = min(ROWS, item.ntok * p.G);
  // partial results: [slot0 + split][kv head][row]
  const size_t slab0 = ((size_t)slot0 * p.KV + g) * ROWS;
  const size_t slab_step = (size_t)p.KV * ROWS;                       // from one split to the next
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
    if (nsplit == 1) {
      const int tok = r / p.G, hh = r - tok * p.G;
      p.out[(size_t)(item.row0 + tok) * p.out_stride + (size_t)(g * p.G + hh) * p.hs + d] =
          __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      const size_t slab = slab0 + (size_t)split * slab_step + r;
      __stcg(p.part_o + slab * p.hs + d, acc);
      if (d == 0) { __stcg(p.part_ml + slab * 2, M); __stcg(p.part_ml + slab * 2 + 1, L); }
    }
  }
  if (nsplit == 1) return;

  // ticket: the last block of this (item, kv head) merges the splits
  __threadfence();
  asm volatile("bar.sync 1, 128;\n" ::: "memory");
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(p.counters + item_idx * p.KV + g, 1);
    s_last = ticket == nsplit - 1;
  }
  asm volatile("bar.sync 1, 128;\n" ::: "memory");
  if (!s_last) return;
  __threadfence();
  // The merge reads nsplit partial results per output. Loads that follow one another in a loop would each
  // cost a trip to L2, so (1) the maxima and sums of all splits come into shared memory in one pass,
  // (2) one thread per row turns them into the weights of the splits and the row's sum, and (3) the
  // outputs are summed over the splits eight loads at a time. (The warps' merge buffers are free by now.)
  float* w_s = reinterpret_cast<float*>(smem_raw);              // [rows_used][nsplit] maxima, then weights
  float* l_s = w_s + rows_used * nsplit;                        // [rows_used][nsplit] sums
  float* L_s = l_s + rows_used * nsplit;                        // [rows_used]
  for (int i = threadIdx.x; i < rows_used * nsplit; i += THREADS) {
    const int r = i / nsplit, sp = i - r * nsplit;
    const size_t slab = slab0 + (size_t)sp * slab_step + r;
    w_s[i] = __ldcg(p.part_ml + slab * 2);
    l_s[i] = __ldcg(p.part_ml + slab * 2 + 1);
  }
  asm volatile("bar.sync 1, 128;\n" ::: "memory");
  for (int r = threadIdx.x; r < rows_used; r += THREADS) {
    float M = -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) M = fmaxf(M, w_s[r * nsplit + sp]);
    float L = 0.f;
    for (int sp = 0; sp < nsplit; ++sp) {
      const float ms = w_s[r * nsplit + sp];
      const float wgt = ms == -INFINITY ? 0.f : exp2f(ms - M);
      L += l_s[r * nsplit + sp] * wgt;
      w_s[r * nsplit + sp] = wgt;
    }
    L_s[r] = L;
  }
  asm volatile("bar.sync 1, 128;\n" ::: "memory");
  // four outputs a thread, sixteen 16-byte loads in flight: with a few rows (a decode step) every thread has
  // one turn, and the splits cost two round trips to L2 instead of one for every eight scalar loads
  const int hs4 = p.hs >> 2;
  for (int idx = threadIdx.x; idx < rows_used * hs4; idx += THREADS) {
    const int r = idx / hs4, d = (idx - r * hs4) << 2;
    const float* src = p.part_o + (slab0 + r) * p.hs + d;       // split sp lies sp * slab_step * hs further
    const size_t step = slab_step * p.hs;
    const float* wr = w_s + r * nsplit;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < nsplit; sp += 16) {
      float4 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        v[u] = sp + u < nsplit ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + u) * step))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 16; ++u)
        if (sp + u < nsplit) {                                   // in the order of the splits
          const float wgt = wr[sp + u];
          acc.x += v[u].x * wgt; acc.y += v[u].y * wgt; acc.z += v[u].z * wgt; acc.w += v[u].w * wgt;
        }
    }
    const float L = L_s[r];
    const int tok = r / p.G, hh = r - tok * p.G;
    bf16* dst = p.out + (size_t)(item.row0 + tok) * p.out_stride + (size_t)(g * p.G + hh) * p.hs + d;
    dst[0] = __float2bfloat16_rn(L > 0.f ? acc.x / L : 0.f);
    dst[1] = __float2bfloat16_rn(L > 0.f ? acc.y / L : 0.f);
    dst[2] = __float2bfloat16_rn(L > 0.f ? acc.z / L : 0.f);
    dst[3] = __float2bfloat16_rn(L > 0.f ? acc.w / L : 0.f);
  }
  if (threadIdx.x == 0) p.counters[item_idx * p.KV + g] = 0;      // ready for the next launch
}

// ---- host side --------------------------------------------------------------------------------
static int rows_for(int H, int KV) {
  const int G = H / KV;
  return G <= 16 ? 16 : (G <= 32 ? 32 : 0);
}

// 1 when the TMA decode kernel takes this layout.
SI_EXPORT int si_attn_decode_tma_ok(int H, int KV, int hs, int page_size) {
  if (KV <= 0 || H % KV) return 0;
  if (hs != 64 && hs != 128) return 0;
  if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return 0;
  return rows_for(H, KV) > 0 && si_encode_fn() != nullptr;
}

SI_EXPORT int si_attn_decode_tma_rows(int H, int KV) { return rows_for(H, KV); }

// Describe one layer's K (or V) cache, [num_pages, KV, page_size, hs] bf16, as the 2-D tensor
// [num_pages * KV * page_size, hs] with boxes of [page_size, 64]. `map_out`: 128 bytes, 64-byte aligned.
SI_EXPORT int si_attn_encode_cache_map(void* map_out, const void* cache, long long num_pages, int KV,
                                       int page_size, int hs) {
  const unsigned long long rows = (unsigned long long)num_pages * KV * page_size;
  if (rows >= (1ull << 31)) return -2;
  return si_encode_bf16_2d((CUtensorMap*)map_out, cache, rows, (unsigned long long)hs, (unsigned long long)hs,
                           (unsigned)page_size);
}

SI_EXPORT long long si_attn_decode_tma_scratch_floats(int num_items, int H, int KV, int hs, int nsplit) {
  if (nsplit <= 1) return 0;
  const long long rows = rows_for(H, KV);
  return SI_ATTN_TICKETS + (long long)num_items * KV * nsplit * rows * (hs + 2);
}

// Scratch of the launch with a work list: the tickets, then `slots` partial results (one per work entry).
SI_EXPORT long long si_attn_decode_tma_work_floats(int slots, int H, int KV, int hs) {
  const long long rows = rows_for(H, KV);
  return SI_ATTN_TICKETS + (long long)slots * KV * rows * (hs + 2);
}

template <int NH, int MT, bool SWAP = false>
static int launch(const AttnParams& p, const CUtensorMap& km, const CUtensorMap& vm, int num_items, int log2_page,
                  const int4* work, int num_work, cudaStream_t stream) {
  constexpr int STAGES = 3, ROWS = 16 * MT, HS_PAD = NH * 64;
  size_t smem = (size_t)(2 * STAGES * 64 + ROWS) * HS_PAD * sizeof(bf16);
  const size_t merge = (size_t)4 * ROWS * (2 + HS_PAD + 4) * sizeof(float);
  if (merge > smem) smem = merge;
  smem += 1024;                                   // room to align the tiles to 1024 bytes
  auto k = attn_decode_tma_kernel<NH, MT, STAGES, SWAP>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const dim3 grid = work ? dim3(num_work, p.KV, 1) : dim3(num_items, p.KV, p.nsplit);
  si_launch(k, grid, dim3(160), smem, stream, p, km, vm, log2_page, work,
            si_pdl_trigger_mode((long long)grid.x * grid.y * grid.z, 2 * si_sm_count()) == 1 ? 1 : 0);
  return si_last_error();
}

// Same contract as si_attn_decode, with the tensor maps of this layer's K and V cache. `max_rows`: the most
// rows (tokens x query heads of a KV head) that any item has, when the caller knows it, else 0; items of at
// most 8 rows take the kernel with the swapped products.
// `work` (may be null): `num_work` entries (item, split, splits of that item, first slot of that item), one
// block row each, so that every item is cut into its own number of shares; entries with item -1 do nothing.
// The splits of an item take the slots first slot .. first slot + splits - 1, all below `work_slots`, and
// every split of an item with more than one has an entry. `nsplit` is not used then; `scratch` holds
// si_attn_decode_tma_work_floats(work_slots, ...) floats.
SI_EXPORT int si_attn_decode_tma(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                 const void* kmap, const void* vmap, const int* block_table, int table_width,
                                 const void* items, int num_items, void* out, long long out_stride, int num_pages,
                                 int page_size, int num_seqs, int H, int KV, int hs, float scale, int window,
                                 int nsplit, const int* work, int num_work, int work_slots, float* scratch,
                                 int max_rows, int* status, cudaStream_t stream) {
  if (num_items <= 0) return 0;
  if (!si_attn_decode_tma_ok(H, KV, hs, page_size) || !kmap || !vmap) return -2;
  if (work) {
    if (num_work <= 0 || work_slots <= 0 || !scratch || ((uintptr_t)work % 16)) return -2;
    nsplit = 1;
  }
  if ((q_stride % 8) || nsplit < 1 || nsplit > 128) return -2;     // the merge stages 2 * rows * nsplit floats in shared memory
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
  p.window = window; p.nsplit = nsplit; p.status = status;
  const int rows = rows_for(H, KV);
  if (nsplit > 1 || work) {
    if (!scratch || (long long)num_items * KV > SI_ATTN_TICKETS) return -2;
    const size_t slots = work ? (size_t)work_slots : (size_t)num_items * nsplit;
    p.counters = reinterpret_cast<int*>(scratch);
    p.part_o = scratch + SI_ATTN_TICKETS;
    p.part_ml = p.part_o + slots * KV * rows * hs;
  }
  const int4* wl = reinterpret_cast<const int4*>(work);
  int log2_page = 0;
  while ((1 << log2_page) < page_size) ++log2_page;
  const CUtensorMap& km = *(const CUtensorMap*)kmap;
  const CUtensorMap& vm = *(const CUtensorMap*)vmap;
  if (rows == 16 && max_rows >= 1 && max_rows <= 8)
    return hs == 64 ? launch<1, 1, true>(p, km, vm, num_items, log2_page, wl, num_work, stream)
                    : launch<2, 1, true>(p, km, vm, num_items, log2_page, wl, num_work, stream);
  if (hs == 64) return rows == 16 ? launch<1, 1>(p, km, vm, num_items, log2_page, wl, num_work, stream)
                                  : launch<1, 2>(p, km, vm, num_items, log2_page, wl, num_work, stream);
  return rows == 16 ? launch<2, 1>(p, km, vm, num_items, log2_page, wl, num_work, stream)
                    : launch<2, 2>(p, km, vm, num_items, log2_page, wl, num_work, stream);
}
