// bf16 matrix product for up to 128 rows (decode batches, short prompt portions, the rows of a mixed step):
// out[m, n] = sum_k x[m, k] * W[n, k], fp32 accumulation in tensor memory, bf16 or fp32 output. The reference
// sends every product to cuBLAS (src/source/op/kernels/cuda/matmul_kernel.cu:128-150). With so few rows the
// product is one pass over the weight matrix, so the kernel is built as a stream of W through the SMs:
//
// * The product is taken the other way round: the 128 rows of a W tile are the M of tcgen05.mma and the rows
//   of x (padded to a multiple of 16) its N, so a full-height instruction is fed by W alone and no tensor-core
//   row is spent on padding. The accumulator holds out^T: tensor-memory lane = output column n, column = row m.
// * One block takes one tile of 128 output columns. A block needs 97 KB of shared memory and 128 columns of
//   tensor memory, so two fit an SM: 224 tiles (the gate/up product of the 8B shape) all run at once and share
//   the memory bandwidth evenly, as the blocks of the few-row kernel do. Where the tiles alone do not fill the
//   GPU, the k range of a tile is cut over the 2 to 8 blocks of a cluster, which add their partial sums up
//   through distributed shared memory: every block writes its accumulator to its own shared memory, the cluster
//   meets at its barrier, and block r of the cluster adds the r-th part of the rows over all blocks, in the
//   order of the blocks, and stores it. Nothing goes through global memory and nobody polls; the only waits
//   are on the block's own barriers, and bounded (SI_WAIT_LIMIT in the status word), and every thread reaches
//   both cluster barriers whatever its waits returned.
//   The cut depends on N and K only, never on the number of rows: a row's result does not depend on what else
//   is in the batch.
// * Warp 0 is the TMA producer (a [128, 64] box of W and a [rows, 64] box of x per k step into a ring of as many
//   stages as 96 KB hold, 128-byte swizzle), warp 1 issues tcgen05.mma, warps 2-5 take the finished accumulator
//   out of tensor memory, 32 rows of x at a time, and store it transposed: for one row the 32 lanes of a warp
//   hold 32 consecutive output columns.
// * W does not depend on the kernel before this one: the producer fetches the W boxes of its first stages
//   before it waits for that kernel (programmatic dependent launch), x after.
// With SWIGLU, W is the stacked gate/up projection interleaved in groups of 8 rows (8 gates, their 8 ups):
// a gate's up sits 8 lanes further, and out[m, f] = silu(gate) * up is stored, [M, N / 2].
// (An earlier kernel cut the stream of (tile, k step) pairs into equal shares over one block an SM and merged
// the partial tiles through global memory by ticket: correct, and slower than this one at every shape but the
// widest, because a partial tile took 3.5 us to hand over and 7 us to add up.)
#include "tma_common.cuh"

typedef __nv_bfloat16 bf16;

#define SI_ROWS_MAX 128                 // rows of x one call takes
#define SI_ROWS_MAX_TILES 16384         // tiles of 128 output columns a call may have (2 M columns)
// A block of a cluster never holds fewer k steps than this (a shorter share would not pay for its start).
#define SI_ROWS_MIN_STEPS 16

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

__device__ __forceinline__ float ld_cluster_f32(unsigned cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}
__device__ __forceinline__ unsigned cluster_size_x() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_nctaid.x;\n" : "=r"(r));
  return r;
}

#define SI_ROWS_TILE_SMEM (96 * 1024)     // operand stages of a block; two blocks fit an SM
#define SI_ROWS_TILE_MAX_STAGES 8

// Stages of [128 x 64] of W and [mpad x 64] of x that fit a block's shared memory.
__host__ __device__ inline int rows_tile_stages(int mpad) {
  const int n = SI_ROWS_TILE_SMEM / (128 * 64 * 2 + mpad * 64 * 2);
  return n < SI_ROWS_TILE_MAX_STAGES ? n : SI_ROWS_TILE_MAX_STAGES;
}

template <typename TO, bool SWIGLU>
__global__ void __launch_bounds__(192, 2)
gemm_rows_tile_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                      TO* __restrict__ out, long long ldo, int M, int N, int K, int* status) {
  constexpr int BN = 128, BK = 64, MAX_STAGES = SI_ROWS_TILE_MAX_STAGES;
  constexpr int W_BYTES = BN * BK * 2;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t acc_full;
  __shared__ unsigned tmem_slot;
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mpad = (M + 15) & ~15;
  const unsigned x_bytes = (unsigned)mpad * BK * 2;
  const int X_BYTES = (int)x_bytes;                        // a multiple of 2 KB: whole swizzle groups of 8 rows
  const int STAGES = rows_tile_stages(mpad);
  unsigned char* Ws = smem;
  unsigned char* Xs = smem + STAGES * W_BYTES;
  float* partial = reinterpret_cast<float*>(smem);        // [mpad][128] once the operands are used up (at most 64 KB)
  const int nk = (K + BK - 1) / BK;
  const int parts = (int)cluster_size_x();                  // blocks that share a tile
  const int part = (int)cluster_cta_rank();
  const int tile = blockIdx.x / parts;
  const int k0 = (int)((long long)nk * part / parts), k1 = (int)((long long)nk * (part + 1) / parts);
  const int steps = k1 - k0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 128);
  tc05_fence_before_sync();
  __syncthreads();
  tc05_fence_after_sync();
  const unsigned tmem = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int ahead = steps < STAGES ? steps : STAGES;    // W does not depend on the kernel before this one
      for (int i = 0; i < ahead; ++i) {
        mbar_expect_tx(&full_bar[i], W_BYTES + x_bytes);
        tma_load_2d(Ws + i * W_BYTES, &wmap, &full_bar[i], (k0 + i) * BK, tile * BN);
      }
      pdl_wait();
      for (int it = 0; it < steps; ++it) {
        const int s = it % STAGES;
        if (it >= STAGES) {
          if (!mbar_wait(&empty_bar[s], (unsigned)(((it / STAGES) - 1) & 1))) {
            set_status(status, SI_WAIT_LIMIT);
            break;
          }
          mbar_expect_tx(&full_bar[s], W_BYTES + x_bytes);
          tma_load_2d(Ws + s * W_BYTES, &wmap, &full_bar[s], (k0 + it) * BK, tile * BN);
        }
        tma_load_2d(Xs + s * X_BYTES, &xmap, &full_bar[s], (k0 + it) * BK, 0);
      }
    }
  } else if (warp == 1) {
    const unsigned idesc = umma_idesc_bf16(BN, mpad, false);
    const unsigned long long wd0 = umma_desc_sw128(Ws, 16, 1024), xd0 = umma_desc_sw128(Xs, 16, 1024);
    bool ok = true;
    for (int it = 0; it < steps && ok; ++it) {
      const int s = it % STAGES;
      ok = mbar_wait_warp(&full_bar[s], (unsigned)((it / STAGES) & 1));
      if (!ok) break;
      tc05_fence_after_sync();
      const unsigned long long wd = wd0 + (unsigned)s * (W_BYTES / 16), xd = xd0 + (unsigned)s * (X_BYTES / 16);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          tc05_mma_bf16(tmem, wd + 2 * k, xd + 2 * k, idesc, (it != 0 || k != 0) ? 1u : 0u);
        tc05_commit(&empty_bar[s]);
        if (it + 1 == steps) tc05_commit(&acc_full);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) set_status(status, SI_WAIT_LIMIT);
  } else {
    pdl_wait();                                           // `out` may still be read by the kernel before
    const int q = warp & 3;                               // tensor-memory lanes q*32 .. q*32+31 = columns of the tile
    const int n = tile * BN + q * 32 + lane;
    bool ok = steps > 0 && mbar_wait_warp(&acc_full, 0);
    if (!ok && steps > 0 && lane == 0) set_status(status, SI_WAIT_LIMIT);
    tc05_fence_after_sync();
    const unsigned src = tmem + ((unsigned)(q * 32) << 16);
#pragma unroll 1
    for (int m0 = 0; m0 < mpad; m0 += 32) {
      float v[32];
      if (ok) {
        tmem_ld_32x32(src + m0, v);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
      }
      if (parts == 1) {
        if (ok) rows_store_chunk<TO, SWIGLU>(out, ldo, v, m0, M, N, n, tile * BN + q * 32, lane);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (m0 + j < mpad) partial[(size_t)(m0 + j) * BN + q * 32 + lane] = v[j];
      }
    }
  }
  if (parts > 1) {
    // every block's partial sum is in its shared memory: the cluster meets, block `part` adds its rows up over
    // all blocks in their order, and the cluster meets again before any block, and its shared memory, goes
    __syncwarp();
    cluster_sync_all();
    if (warp >= 2) {
      const int q = warp & 3;
      const int n = tile * BN + q * 32 + lane;
      const int lo = mpad * part / parts, hi = mpad * (part + 1) / parts;
#pragma unroll 1
      for (int m0 = lo; m0 < hi; m0 += 32) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
        for (int c = 0; c < parts; ++c) {
          const unsigned theirs = cluster_map_u32(partial + q * 32 + lane, (unsigned)c);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (m0 + j < hi) v[j] += ld_cluster_f32(theirs + (unsigned)((m0 + j) * BN * 4));
        }
        rows_store_chunk<TO, SWIGLU>(out, ldo, v, m0, M < hi ? M : hi, N, n, tile * BN + q * 32, lane);
      }
    }
    cluster_sync_all();
  }
  tc05_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 128);
}

// Blocks that share a tile of the tile-a-block kernel: as many as still fit the GPU at two blocks an SM, at most
// eight (a portable cluster), none with fewer than SI_ROWS_MIN_STEPS k steps. Depends on N and K only.
static int rows_ksplit(int N, int K) {
  const int tiles = (N + 127) / 128, nk = (K + 63) / 64;
  if (const char* e = getenv("SI_ROWS_KSPLIT")) {          // for measurements
    const int c = atoi(e);
    if (c >= 1 && c <= 8 && c <= nk) return c;
  }
  int c = 1;
  while (c < 8 && (long long)tiles * (c + 1) <= 2LL * si_sm_count() && nk / (c + 1) >= SI_ROWS_MIN_STEPS) ++c;
  return c;
}

template <typename TO, bool SWIGLU>
static int rows_tile_launch(const CUtensorMap& xm, const void* wmap, void* out, long long ldo, int M, int N, int K,
                            int* status, cudaStream_t stream) {
  const size_t smem = SI_ROWS_TILE_SMEM + 1024;
  auto k = gemm_rows_tile_kernel<TO, SWIGLU>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int parts = rows_ksplit(N, K);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(((N + 127) / 128) * parts));
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)parts;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = si_pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, k, xm, *(const CUtensorMap*)wmap, (TO*)out, ldo, M, N, K, status);
  return si_last_error();
}

SI_EXPORT int si_gemm_rows_max_rows() { return SI_ROWS_MAX; }

template <typename TO, bool SWIGLU>
static int rows_launch(const void* x, long long ldx, const void* wmap, void* out, long long ldo, int M, int N, int K,
                       int* status, cudaStream_t stream) {
  if (M > SI_ROWS_MAX || K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)x % 16) || !wmap) return -2;
  if ((N + 127) / 128 > SI_ROWS_MAX_TILES) return -2;
  CUtensorMap xm;
  const int mpad = (M + 15) & ~15;
  const int rc = si_encode_bf16_2d(&xm, x, (unsigned long long)M, (unsigned long long)K, (unsigned long long)ldx, (unsigned)mpad);
  if (rc) return rc;
  return rows_tile_launch<TO, SWIGLU>(xm, wmap, out, ldo, M, N, K, status, stream);
}

// x: [M, K] bf16 rows `ldx` apart, M <= 128. `wmap`: the weight's tensor map with boxes of [128, 64]
// (si_gemm_tc05_encode_weight with box_rows 128). out_dtype: SI_BF16 or SI_F32. Returns 0, a CUDA error code, or
// -2 (sizes refused).
SI_EXPORT int si_gemm_rows(const void* x, long long ldx, const void* wmap, void* out, long long ldo, int out_dtype,
                           int M, int N, int K, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (out_dtype == SI_BF16) return rows_launch<bf16, false>(x, ldx, wmap, out, ldo, M, N, K, status, stream);
  return rows_launch<float, false>(x, ldx, wmap, out, ldo, M, N, K, status, stream);
}

// out[M, F] = silu(gate) * up (bf16) of the stacked projection x[M, K] W[2F, K]^T, rows of W interleaved in
// groups of 8; F a multiple of 8.
SI_EXPORT int si_gemm_rows_swiglu(const void* x, long long ldx, const void* wmap, void* out, long long ldo,
                                  int M, int F, int K, int* status, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return 0;
  if (F % 8) return -2;
  return rows_launch<bf16, true>(x, ldx, wmap, out, ldo, M, 2 * F, K, status, stream);
}
