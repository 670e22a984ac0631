// bf16 matrix product for up to 128 rows (decode batches, short prompt portions, the rows of a mixed step):
// out[m, n] = sum_k x[m, k] * W[n, k], fp32 accumulation in tensor memory, bf16 or fp32 output. The reference
// sends every product to cuBLAS (src/source/op/kernels/cuda/matmul_kernel.cu:128-150). With so few rows the
// product is one pass over the weight matrix, so the kernel is built as a stream of W through the SMs:
//
// * The product is taken the other way round: the 128 rows of a W tile are the M of tcgen05.mma and the rows
//   of x (padded to a multiple of 16) its N, so a full-height instruction is fed by W alone and no tensor-core
//   row is spent on padding. The accumulator holds out^T: tensor-memory lane = output column n, column = row m.
// * The work is the list of (tile of 128 output columns, k step of 64) pairs in that order, cut into as many
//   equal contiguous shares as there are blocks (one per SM): every block streams the same number of bytes,
//   whatever the number of tiles. A share that starts or ends inside a tile computes a partial sum of that
//   tile, writes it to a slot of `scratch` and takes a ticket of that tile; the block that takes the tile's
//   last ticket adds the partial sums up, in the order of the blocks (not of their arrival), and stores the
//   tile. Nobody waits for another block; the only waits are on the block's own barriers, and bounded
//   (SI_WAIT_LIMIT in the status word).
//   The cut depends on N and K and the number of blocks only, never on the number of rows: a row's result
//   does not depend on what else is in the batch.
// * Warp 0 is the TMA producer (a [128, 64] box of W and a [rows, 64] box of x per k step into a ring of six
//   stages, 128-byte swizzle), warp 1 issues tcgen05.mma into one of two accumulators, warps 2-5 take a
//   finished accumulator out of tensor memory, 32 rows of x at a time, and store it transposed: for one row
//   the 32 lanes of a warp hold 32 consecutive output columns.
// * W does not depend on the kernel before this one: the producer fetches the W boxes of its first stages
//   before it waits for that kernel (programmatic dependent launch), x after.
// With SWIGLU, W is the stacked gate/up projection interleaved in groups of 8 rows (8 gates, their 8 ups):
// a gate's up sits 8 lanes further, and out[m, f] = silu(gate) * up is stored, [M, N / 2].
#include "tma_common.cuh"

typedef __nv_bfloat16 bf16;

#define SI_ROWS_MAX 128                 // rows of x one call takes
#define SI_ROWS_SLOT_FLOATS (128 * 128) // one block's partial sum: [row][column of the tile]
#define SI_ROWS_MAX_TILES 16384         // tiles of 128 output columns a call may have (2 M columns)

// A share never holds fewer k steps than this (a block whose share is shorter would not pay for its start).
#define SI_ROWS_MIN_STEPS 8

__host__ __device__ inline long long rows_share_start(long long units, int blocks, int c) {
  return units * c / blocks;
}
// The block whose share holds unit u.
__device__ inline int rows_block_of(long long units, int blocks, long long u) {
  int c = (int)((u * blocks) / units);
  while (c + 1 < blocks && rows_share_start(units, blocks, c + 1) <= u) ++c;
  while (c > 0 && rows_share_start(units, blocks, c) > u) --c;
  return c;
}

template <typename TO> __device__ __forceinline__ void rows_store(TO* p, float v);
template <> __device__ __forceinline__ void rows_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void rows_store<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// 32 rows of this thread's output column: `n` the column, `base` the first column of the warp's 32.
template <typename TO, bool SWIGLU>
__device__ __forceinline__ void rows_store_chunk(TO* __restrict__ out, long long ldo, float (&v)[32], int m0, int M, int N,
                                                 int n, int base, int lane) {
  if (SWIGLU) {
    bf16* o = (bf16*)out;
    const int f = base / 2 + (lane >> 4) * 8 + (lane & 7);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float up = __shfl_down_sync(0xffffffffu, v[j], 8);
      if ((lane & 8) == 0 && m0 + j < M && n + 8 < N)
        o[(size_t)(m0 + j) * ldo + f] = __float2bfloat16_rn(silu_mul(
            __bfloat162float(__float2bfloat16_rn(v[j])), __bfloat162float(__float2bfloat16_rn(up))));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (m0 + j < M && n < N) rows_store<TO>(out + (size_t)(m0 + j) * ldo + n, v[j]);
  }
}

// Built with -DSI_ROWS_TIMING, every block leaves the times (ns, %globaltimer) of its milestones in
// g_rows_times, which si_gemm_rows_times() copies out: where a launch spends its time, block by block.
#ifdef SI_ROWS_TIMING
__device__ unsigned long long g_rows_times[8][256][8];   // the last eight launches
__device__ unsigned g_rows_seq, g_rows_done;
__device__ __forceinline__ void rows_stamp(int i) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  g_rows_times[*(volatile unsigned*)&g_rows_seq % 8][blockIdx.x][i] = t;
}
#else
__device__ __forceinline__ void rows_stamp(int) {}
#endif

template <int STAGES, typename TO, bool SWIGLU>
__global__ void __launch_bounds__(192)
gemm_rows_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                 TO* __restrict__ out, long long ldo, int M, int N, int K, float* __restrict__ scratch,
                 int* __restrict__ tickets, int* status) {
  constexpr int BN = 128, BK = 64;                         // output columns a tile, k a step
  constexpr int W_BYTES = BN * BK * 2, X_BYTES = SI_ROWS_MAX * BK * 2;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_slot;
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* Ws = smem;
  unsigned char* Xs = smem + STAGES * W_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mpad = (M + 15) & ~15;                          // the N of the instruction
  const unsigned x_bytes = (unsigned)mpad * BK * 2;
  const int n_tiles = (N + BN - 1) / BN, nk = (K + BK - 1) / BK;
  const long long units = (long long)n_tiles * nk;
  const int blocks = gridDim.x, me = blockIdx.x;
  const long long u0 = rows_share_start(units, blocks, me), u1 = rows_share_start(units, blocks, me + 1);
  if (threadIdx.x == 0) rows_stamp(0);

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
#pragma unroll
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 256);               // two accumulators of up to 128 columns
  tc05_fence_before_sync();
  __syncthreads();
  tc05_fence_after_sync();
  const unsigned tmem = tmem_slot;
  if (threadIdx.x == 0) rows_stamp(1);

  if (warp == 0) {
    if (lane == 0) {
      // W boxes of the first stages go out before the wait for the kernel that made x
      const long long ahead = u1 - u0 < STAGES ? u1 - u0 : STAGES;
      for (long long i = 0; i < ahead; ++i) {
        const long long u = u0 + i;
        const int tile = (int)(u / nk), kb = (int)(u - (long long)tile * nk);
        mbar_expect_tx(&full_bar[i], W_BYTES + x_bytes);
        tma_load_2d(Ws + i * W_BYTES, &wmap, &full_bar[i], kb * BK, tile * BN);
      }
      pdl_wait();
      bool ok = true;
      long long it = 0;
      for (long long u = u0; u < u1 && ok; ++u, ++it) {
        const int s = (int)(it % STAGES);
        const int tile = (int)(u / nk), kb = (int)(u - (long long)tile * nk);
        if (it >= STAGES) {
          if (!mbar_wait(&empty_bar[s], (unsigned)(((it / STAGES) - 1) & 1))) {
            set_status(status, SI_WAIT_LIMIT);
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], W_BYTES + x_bytes);
          tma_load_2d(Ws + s * W_BYTES, &wmap, &full_bar[s], kb * BK, tile * BN);
        }
        tma_load_2d(Xs + s * X_BYTES, &xmap, &full_bar[s], kb * BK, 0);
      }
    }
  } else if (warp == 1) {
    const unsigned idesc = umma_idesc_bf16(BN, mpad, false);
    const unsigned long long wd0 = umma_desc_sw128(Ws, 16, 1024), xd0 = umma_desc_sw128(Xs, 16, 1024);
    bool ok = true;
    long long it = 0;
    int local = 0;
    for (long long u = u0; u < u1 && ok; ++local) {
      const int tile = (int)(u / nk);
      const long long seg_end = (long long)(tile + 1) * nk < u1 ? (long long)(tile + 1) * nk : u1;
      const int buf = local & 1;
      if (local >= 2) ok = mbar_wait_warp(&acc_empty[buf], (unsigned)(((local >> 1) - 1) & 1));
      if (!ok) break;
      tc05_fence_after_sync();
      const unsigned acc = tmem + buf * SI_ROWS_MAX;
      for (bool first = true; u < seg_end; ++u, ++it, first = false) {
        const int s = (int)(it % STAGES);
        ok = mbar_wait_warp(&full_bar[s], (unsigned)((it / STAGES) & 1));
        if (!ok) break;
        if (it == 0 && lane == 0) rows_stamp(2);
        tc05_fence_after_sync();
        const unsigned long long wd = wd0 + (unsigned)s * (W_BYTES / 16), xd = xd0 + (unsigned)s * (X_BYTES / 16);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc05_mma_bf16(acc, wd + 2 * k, xd + 2 * k, idesc, (!first || k != 0) ? 1u : 0u);
          tc05_commit(&empty_bar[s]);
          if (u + 1 == seg_end) tc05_commit(&acc_full[buf]);
        }
        __syncwarp();
      }
    }
    if (!ok && lane == 0) set_status(status, SI_WAIT_LIMIT);
    if (lane == 0) rows_stamp(3);
  } else {
    pdl_wait();                                           // `out` and `scratch` may still be read by the kernel before
    const int q = warp & 3;                               // tensor-memory lanes q*32 .. q*32+31 = columns of the tile
    int local = 0;
    for (long long u = u0; u < u1; ++local) {
      const int tile = (int)(u / nk);
      const long long t0 = (long long)tile * nk, t1 = t0 + nk;
      const long long seg_end = t1 < u1 ? t1 : u1;
      const bool whole = (u == t0) && seg_end == t1;
      const int buf = local & 1;
      u = seg_end;
      if (!mbar_wait_warp(&acc_full[buf], (unsigned)((local >> 1) & 1))) {
        if (lane == 0) set_status(status, SI_WAIT_LIMIT);
        break;
      }
      tc05_fence_after_sync();
      if (q == 0 && lane == 0) rows_stamp(local == 0 ? 4 : 6);
      const int n = tile * BN + q * 32 + lane;            // this thread's output column
      const unsigned src = tmem + ((unsigned)(q * 32) << 16) + (unsigned)(buf * SI_ROWS_MAX);
      // a share's first segment goes to the block's first slot, a later one (its last) to the second
      float* mine = scratch + (size_t)(2 * me + (local == 0 ? 0 : 1)) * SI_ROWS_SLOT_FLOATS + q * 32 + lane;
#pragma unroll 1
      for (int m0 = 0; m0 < mpad; m0 += 32) {
        float v[32];
        tmem_ld_32x32(src + m0, v);
        if (m0 + 32 >= mpad) {                             // the accumulator is in registers: hand it back
          tc05_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (whole) {
          rows_store_chunk<TO, SWIGLU>(out, ldo, v, m0, M, N, n, tile * BN + q * 32, lane);
        } else {                                           // a partial sum: [row][column], this warp's 32 columns
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (m0 + j < mpad) __stcg(mine + (size_t)(m0 + j) * BN, v[j]);
        }
      }
      if (whole) continue;
      // The partial sum is written. Whoever comes last to a tile adds the partial sums up, in the order of the
      // blocks, whichever block it is itself: nobody waits for anybody. One ticket counter per (tile, warp).
      __threadfence();
      __syncwarp();
      const int c_first = rows_block_of(units, blocks, t0), c_last = rows_block_of(units, blocks, t1 - 1);
      int* ticket = tickets + (size_t)tile * 4 + q;
      int mine_is_last = 0;
      if (lane == 0) mine_is_last = atomicAdd(ticket, 1) == c_last - c_first;
      if (!__shfl_sync(0xffffffffu, mine_is_last, 0)) continue;
      __threadfence();
      if (q == 0 && lane == 0) rows_stamp(5);
#pragma unroll 1
      for (int m0 = 0; m0 < mpad; m0 += 32) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
#pragma unroll 1
        for (int c = c_first; c <= c_last; c += 4) {       // four partial sums in flight at a time
          float t[4][32];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int ci = c + i <= c_last ? c + i : c_last;
            const int slot = 2 * ci + (rows_share_start(units, blocks, ci) >= t0 ? 0 : 1);
            const float* theirs = scratch + (size_t)slot * SI_ROWS_SLOT_FLOATS + q * 32 + lane + (size_t)m0 * BN;
#pragma unroll
            for (int j = 0; j < 32; ++j) t[i][j] = (m0 + j < mpad) ? __ldcg(theirs + (size_t)j * BN) : 0.f;
          }
          asm volatile("" ::: "memory");                   // every load above is issued before the first sum waits
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (c + i <= c_last) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += t[i][j];
            }
        }
        rows_store_chunk<TO, SWIGLU>(out, ldo, v, m0, M, N, n, tile * BN + q * 32, lane);
      }
      __syncwarp();
      if (lane == 0) *ticket = 0;                          // ready for the next launch
    }
  }
  tc05_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) rows_stamp(7);
  if (warp == 1) tmem_dealloc(tmem, 256);
#ifdef SI_ROWS_TIMING
  if (threadIdx.x == 0 && atomicAdd(&g_rows_done, 1u) == gridDim.x - 1) {   // the launch's last block
    g_rows_done = 0;
    __threadfence();
    atomicAdd(&g_rows_seq, 1u);
  }
#endif
}

#ifdef SI_ROWS_TIMING
SI_EXPORT int si_gemm_rows_times(unsigned long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_rows_times, sizeof(g_rows_times));
}
#endif

static int rows_blocks(int N, int K) {
  const long long units = (long long)((N + 127) / 128) * ((K + 63) / 64);
  if (const char* e = getenv("SI_ROWS_BLOCKS")) {          // for measurements: a fixed number of blocks
    const long long b = atoll(e);
    if (b >= 1 && b <= units && b <= si_sm_count()) return (int)b;
  }
  long long b = units / SI_ROWS_MIN_STEPS;
  if (b < 1) b = 1;
  return (int)(b < si_sm_count() ? b : si_sm_count());
}

// Words (4 bytes) of scratch a call needs, whatever its sizes: two partial sums per block (a share's first and
// last tile), one block per SM, and the tickets, four per tile. The tickets (the last 4 * SI_ROWS_MAX_TILES
// words) must be zero before the first call; calls leave them zero.
SI_EXPORT long long si_gemm_rows_scratch_words() {
  return (long long)si_sm_count() * 2 * SI_ROWS_SLOT_FLOATS + 4 * SI_ROWS_MAX_TILES;
}
SI_EXPORT int si_gemm_rows_max_rows() { return SI_ROWS_MAX; }

template <typename TO, bool SWIGLU>
static int rows_launch(const void* x, long long ldx, const void* wmap, void* out, long long ldo, int M, int N, int K,
                       float* scratch, int* status, cudaStream_t stream) {
  if (M > SI_ROWS_MAX || K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)x % 16) || !wmap || !scratch) return -2;
  if ((N + 127) / 128 > SI_ROWS_MAX_TILES) return -2;
  CUtensorMap xm;
  const int mpad = (M + 15) & ~15;
  const int rc = si_encode_bf16_2d(&xm, x, (unsigned long long)M, (unsigned long long)K, (unsigned long long)ldx, (unsigned)mpad);
  if (rc) return rc;
  constexpr int STAGES = 6;
  const size_t smem = (size_t)STAGES * (128 * 64 * 2 + SI_ROWS_MAX * 64 * 2) + 1024;
  auto k = gemm_rows_kernel<STAGES, TO, SWIGLU>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  int* tickets = reinterpret_cast<int*>(scratch + (size_t)si_sm_count() * 2 * SI_ROWS_SLOT_FLOATS);
  si_launch(k, dim3(rows_blocks(N, K)), dim3(192), smem, stream, xm, *(const CUtensorMap*)wmap, (TO*)out, ldo, M, N, K,
            scratch, tickets, status);
  return si_last_error();
}

// x: [M, K] bf16 rows `ldx` apart, M <= 128. `wmap`: the weight's tensor map with boxes of [128, 64]
// (si_gemm_tc05_encode_weight with box_rows 128). `scratch`: si_gemm_rows_scratch_words() words, shared by all
// calls on one stream. out_dtype: SI_BF16 or SI_F32. Returns 0, a CUDA error code, or -2 (sizes refused).
SI_EXPORT int si_gemm_rows(const void* x, long long ldx, const void* wmap, void* out, long long ldo, int out_dtype,
                           int M, int N, int K, float* scratch, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (out_dtype == SI_BF16) return rows_launch<bf16, false>(x, ldx, wmap, out, ldo, M, N, K, scratch, status, stream);
  return rows_launch<float, false>(x, ldx, wmap, out, ldo, M, N, K, scratch, status, stream);
}

// out[M, F] = silu(gate) * up (bf16) of the stacked projection x[M, K] W[2F, K]^T, rows of W interleaved in
// groups of 8; F a multiple of 8.
SI_EXPORT int si_gemm_rows_swiglu(const void* x, long long ldx, const void* wmap, void* out, long long ldo,
                                  int M, int F, int K, float* scratch, int* status, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return 0;
  if (F % 8) return -2;
  return rows_launch<bf16, true>(x, ldx, wmap, out, ldo, M, 2 * F, K, scratch, status, stream);
}
