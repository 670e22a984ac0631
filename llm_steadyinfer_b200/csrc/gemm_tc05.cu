// bf16 matrix product on the 5th-generation tensor cores: out[M, N] = x[M, K] * W[N, K]^T with
// fp32 accumulation in tensor memory. The reference leaves every product to cuBLAS
// (src/source/op/kernels/cuda/matmul_kernel.cu:128-150); this is the package's own kernel for
// products with many rows (prompt portions).
//
// Persistent blocks, one per SM, each taking 128 x 256 output tiles in turn (tiles that run at the
// same time share their 256 rows of W, which so comes from HBM once). Warp 0 is the TMA producer:
// per 64-wide k step it fetches a [128, 64] box of x and a [256, 64] box of W (128-byte swizzle)
// into a ring of stages that runs on across tiles. Warp 1 issues tcgen05.mma (four K=16
// instructions of 128 x 256 per stage, descriptors advanced by 32 bytes) into one of two
// accumulators in tensor memory (2 x 256 columns) and releases each stage with tcgen05.commit.
// Warps 2-5 take a finished accumulator out of tensor memory (tcgen05.ld), hand it back as soon as
// it is in registers, and store the rows while the next tile's instructions already run into the
// other accumulator. With SWIGLU the product is the stacked gate/up projection whose rows of W are
// interleaved in groups of 8 (8 gates, their 8 ups, ...): a thread then holds gate and up of the
// same output and stores silu(gate) * up, [M, N/2].
// All waits are bounded; a wait that runs out sets SI_WAIT_LIMIT and the block stops storing.
#include "tma_common.cuh"

typedef __nv_bfloat16 bf16;

template <typename TO> __device__ __forceinline__ void store_row32(TO* dst, const float (&v)[32], int valid, bool vec);
template <> __device__ __forceinline__ void store_row32<float>(float* dst, const float (&v)[32], int valid, bool vec) {
  if (vec && valid == 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (i < valid) dst[i] = v[i];       // unrolled: v stays in registers
  }
}
template <> __device__ __forceinline__ void store_row32<bf16>(bf16* dst, const float (&v)[32], int valid, bool vec) {
  if (vec && valid == 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 raw;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
      reinterpret_cast<uint4*>(dst)[i] = raw;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (i < valid) dst[i] = __float2bfloat16_rn(v[i]);
  }
}

// The residual stream's add in the epilogue: dst (fp32) += the 32 sums, each rounded to bf16 first, as when the
// product is stored in bf16 and the norm kernel after it adds it into the stream.
__device__ __forceinline__ void add_row32(float* dst, const float (&v)[32], int valid, bool vec) {
  if (vec && valid == 32) {
    float4 r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = reinterpret_cast<const float4*>(dst)[i];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      r[i].x += __bfloat162float(__float2bfloat16_rn(v[4 * i]));
      r[i].y += __bfloat162float(__float2bfloat16_rn(v[4 * i + 1]));
      r[i].z += __bfloat162float(__float2bfloat16_rn(v[4 * i + 2]));
      r[i].w += __bfloat162float(__float2bfloat16_rn(v[4 * i + 3]));
      reinterpret_cast<float4*>(dst)[i] = r[i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (i < valid) dst[i] += __bfloat162float(__float2bfloat16_rn(v[i]));
  }
}

// What the epilogue does with a tile: store it, store silu(gate) * up of it, or add it into an fp32 tensor.
enum : int { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_ADD = 2 };

// 16 outputs of the gated activation from 32 accumulator columns (two groups of 8 gates + 8 ups); gate and
// up are rounded to bf16 first, as when the projection is stored and a second kernel applies the activation.
__device__ __forceinline__ void store_swiglu16(bf16* dst, const float (&v)[32], int valid, bool vec) {
  float o[16];
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i)
      o[8 * g + i] = silu_mul(__bfloat162float(__float2bfloat16_rn(v[16 * g + i])), __bfloat162float(__float2bfloat16_rn(v[16 * g + 8 + i])));
  if (vec && valid == 16) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 raw;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(o[8 * i + 2 * j], o[8 * i + 2 * j + 1]);
      reinterpret_cast<uint4*>(dst)[i] = raw;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) if (i < valid) dst[i] = __float2bfloat16_rn(o[i]);
  }
}

template <int STAGES, typename TO, int EPI>
__global__ void __launch_bounds__(192)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
                 TO* __restrict__ out, long long ldo, int M, int N, int K, int* status) {
  constexpr int BM = 128, BN = 256, BK = 64;
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_slot;
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* As = smem;
  unsigned char* Bs = smem + STAGES * A_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  const int nk = (K + BK - 1) / BK;
  pdl_trigger();

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
#pragma unroll
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }   // 4 epilogue warps
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 2 * BN);
  tc05_fence_before_sync();
  __syncthreads();
  tc05_fence_after_sync();
  const unsigned tmem = tmem_slot;
  pdl_wait();                                           // see the pair kernel

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;                                       // k steps issued so far, over all tiles of this block
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], (unsigned)(((it / STAGES) - 1) & 1))) {
            set_status(status, SI_WAIT_LIMIT);
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], A_BYTES + B_BYTES);
          tma_load_2d(As + s * A_BYTES, &amap, &full_bar[s], kb * BK, m0);
          tma_load_2d(Bs + s * B_BYTES, &bmap, &full_bar[s], kb * BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp runs this code and one elected lane issues. An instruction is accepted only as fast as
    // the tensor cores run, so between two of them this warp does as little as it can.
    constexpr unsigned idesc = umma_idesc_bf16(BM, BN, false);
    const unsigned long long ad0 = umma_desc_sw128(As, 16, 1024), bd0 = umma_desc_sw128(Bs, 16, 1024);
    int it = 0, local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      if (local >= 2) ok = mbar_wait_warp(&acc_empty[buf], (unsigned)(((local >> 1) - 1) & 1));
      if (!ok) break;
      tc05_fence_after_sync();
      const unsigned acc = tmem + buf * BN;
      for (int kb = 0; kb < nk; ++kb, ++it) {
        const int s = it % STAGES;
        ok = mbar_wait_warp(&full_bar[s], (unsigned)((it / STAGES) & 1));
        if (!ok) break;
        tc05_fence_after_sync();
        const unsigned long long ad = ad0 + (unsigned)s * (A_BYTES / 16), bd = bd0 + (unsigned)s * (B_BYTES / 16);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc05_mma_bf16(acc, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          tc05_commit(&empty_bar[s]);          // the stage is free once these instructions have read it
          if (kb == nk - 1) tc05_commit(&acc_full[buf]);
        }
        __syncwarp();
      }
    }
    if (!ok && lane == 0) set_status(status, SI_WAIT_LIMIT);
  } else {
    const int q = warp & 3;                   // the 32 tensor-memory lanes this warp may read
    const bool vec = (ldo % 8 == 0) && ((uintptr_t)out % 16 == 0);
    const bool vec4 = (ldo % 4 == 0) && ((uintptr_t)out % 16 == 0);          // rows of fp32 in 16-byte pieces
    int local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
      if (!mbar_wait_warp(&acc_full[buf], (unsigned)((local >> 1) & 1))) {
        if (lane == 0) set_status(status, SI_WAIT_LIMIT);
        break;
      }
      tc05_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const unsigned src = tmem + ((unsigned)(q * 32) << 16) + (unsigned)(buf * BN);
#pragma unroll 1
      for (int h = 0; h < BN / 128; ++h) {
        float v[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32_issue(src + h * 128 + c * 32, v[c]);
        tmem_ld_wait();
        if (h == BN / 128 - 1) {                // the accumulator is in registers: the issuer may have it back
          tc05_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int n = n0 + h * 128 + c * 32;
          if (row < M && n < N) {
            if (EPI == EPI_SWIGLU) store_swiglu16((bf16*)out + (size_t)row * ldo + n / 2, v[c], min(16, (N - n) / 2), vec);
            else if (EPI == EPI_ADD) add_row32((float*)out + (size_t)row * ldo + n, v[c], min(32, N - n), vec4);
            else store_row32<TO>(out + (size_t)row * ldo + n, v[c], min(32, N - n), vec);
          }
        }
      }
    }
  }
  tc05_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 2 * BN);
}


// The same product with two CTAs (a cluster of two, on neighbouring SMs) on one 256 x 256 tile: each CTA fetches
// its 128 rows of x and its 128 of the tile's 256 rows of W per k step (32 KB instead of 48 KB a stage, so six
// stages fit), the leader CTA issues tcgen05.mma.cta_group::2 over both CTAs' shared memory, and each CTA ends
// up with its 128 rows of the accumulator in its own tensor memory, which its four epilogue warps store. Per
// output a CTA reads a third less from L2 and each CTA reads only half of the W tile from shared memory; at the
// power cap, where long products run, that energy is what sets their time. Loads are plain TMA loads, one box per
// CTA, their bytes counted at the leader's barrier; only arrivals are sent to both CTAs (tcgen05.commit).
// Barriers: full[s] (leader: one arrival with the bytes of all four boxes), empty[s] (each CTA: the commit
// after the stage's instructions), acc_full[b] (each CTA: the commit after a tile's last instruction),
// acc_empty[b] (leader: the eight epilogue warps of both CTAs).
template <int STAGES, typename TO, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192)
gemm_tc05_pair_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
                      TO* __restrict__ out, long long ldo, int M, int N, int K, int* status) {
  constexpr int BM = 128, BN = 256, BK = 64;             // BM, and BN / 2 rows of W, per CTA
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_slot;
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* As = smem;
  unsigned char* Bs = smem + STAGES * A_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_cta_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  const int nk = (K + BK - 1) / BK;
  pdl_trigger();                                          // one block an SM: the next kernel's blocks take no block's place

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
#pragma unroll
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }   // 4 epilogue warps of each CTA
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(&tmem_slot, 2 * BN);
  tc05_fence_before_sync();
  cluster_sync_all();                                     // both CTAs' barriers and tensor memory are ready
  tc05_fence_after_sync();
  const unsigned tmem = tmem_slot;
  // Launched as a programmatic dependent: everything above ran while the kernel before this one was ending. W does
  // not depend on that kernel, so the producer also fetches the W boxes of its first stages before it waits;
  // nothing else touches global memory before that kernel's results are there.
  if (warp == 0) {
    if (lane == 0) {
      const long long total = (long long)((tiles - pair + pairs - 1) / pairs) * nk;     // k steps of this pair
      const int ahead = total < STAGES ? (int)total : STAGES;
      for (int i = 0; i < ahead; ++i) {
        const int tile = pair + (i / nk) * pairs, kb = i % nk;
        const int n0 = (tile / m_tiles) * BN + (int)rank * (BN / 2);
        if (rank == 0) mbar_expect_tx(&full_bar[i], 2 * (A_BYTES + B_BYTES));
        tma_load_2d_pair(Bs + i * B_BYTES, &bmap, cluster_map_u32(&full_bar[i], 0), kb * BK, n0);
      }
      pdl_wait();
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs) {
        const int m0 = (tile % m_tiles) * 2 * BM + (int)rank * BM;
        const int n0 = (tile / m_tiles) * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % STAGES;
          const unsigned bar = cluster_map_u32(&full_bar[s], 0);
          if (it >= ahead) {
            if (it >= STAGES && !mbar_wait(&empty_bar[s], (unsigned)(((it / STAGES) - 1) & 1))) {
              set_status(status, SI_WAIT_LIMIT);
              ok = false;
              break;
            }
            if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * (A_BYTES + B_BYTES));
            tma_load_2d_pair(Bs + s * B_BYTES, &bmap, bar, kb * BK, n0);
          }
          tma_load_2d_pair(As + s * A_BYTES, &amap, bar, kb * BK, m0);
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {
      constexpr unsigned idesc = umma_idesc_bf16(2 * BM, BN, false);
      const unsigned long long ad0 = umma_desc_sw128(As, 16, 1024), bd0 = umma_desc_sw128(Bs, 16, 1024);
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs, ++local) {
        const int buf = local & 1;
        if (local >= 2) ok = mbar_wait_warp(&acc_empty[buf], (unsigned)(((local >> 1) - 1) & 1));
        if (!ok) break;
        tc05_fence_after_sync();
        const unsigned acc = tmem + buf * BN;
        for (int kb = 0; kb < nk; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait_warp(&full_bar[s], (unsigned)((it / STAGES) & 1));
          if (!ok) break;
          tc05_fence_after_sync();
          const unsigned long long ad = ad0 + (unsigned)s * (A_BYTES / 16), bd = bd0 + (unsigned)s * (B_BYTES / 16);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              tc05_mma_bf16_pair(acc, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            tc05_commit_pair(&empty_bar[s], 3);     // both CTAs' stages are free once these have read them
            if (kb == nk - 1) tc05_commit_pair(&acc_full[buf], 3);
          }
          __syncwarp();
        }
      }
      if (!ok && lane == 0) set_status(status, SI_WAIT_LIMIT);
    }
  } else {
    pdl_wait();                                           // `out` may still be read by the kernel before this one
    const int q = warp & 3;
    const bool vec = (ldo % 8 == 0) && ((uintptr_t)out % 16 == 0);
    const bool vec4 = (ldo % 4 == 0) && ((uintptr_t)out % 16 == 0);          // rows of fp32 in 16-byte pieces
    int local = 0;
    for (int tile = pair; tile < tiles; tile += pairs, ++local) {
      const int buf = local & 1;
      const int m0 = (tile % m_tiles) * 2 * BM + (int)rank * BM, n0 = (tile / m_tiles) * BN;
      if (!mbar_wait_warp(&acc_full[buf], (unsigned)((local >> 1) & 1))) {
        if (lane == 0) set_status(status, SI_WAIT_LIMIT);
        break;
      }
      tc05_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const unsigned src = tmem + ((unsigned)(q * 32) << 16) + (unsigned)(buf * BN);
#pragma unroll 1
      for (int h = 0; h < BN / 128; ++h) {
        float v[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32_issue(src + h * 128 + c * 32, v[c]);
        tmem_ld_wait();
        if (h == BN / 128 - 1) {                // in registers: the leader's issuer may have the accumulator back
          tc05_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(cluster_map_u32(&acc_empty[buf], 0));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int n = n0 + h * 128 + c * 32;
          if (row < M && n < N) {
            if (EPI == EPI_SWIGLU) store_swiglu16((bf16*)out + (size_t)row * ldo + n / 2, v[c], min(16, (N - n) / 2), vec);
            else if (EPI == EPI_ADD) add_row32((float*)out + (size_t)row * ldo + n, v[c], min(32, N - n), vec4);
            else store_row32<TO>(out + (size_t)row * ldo + n, v[c], min(32, N - n), vec);
          }
        }
      }
    }
  }
  tc05_fence_before_sync();
  cluster_sync_all();                                     // no CTA frees tensor memory the other one's instructions use
  if (warp == 1) tmem_dealloc_pair(tmem, 2 * BN);
}

// SI_GEMM_PAIR=0 in the environment keeps every product on the one-CTA kernel.
static bool pair_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("SI_GEMM_PAIR");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

template <typename TO, int EPI>
static int launch_pair(const CUtensorMap& am, const CUtensorMap& bm_half, void* out, long long ldo, int M, int N, int K,
                       int* status, cudaStream_t stream) {
  constexpr int STAGES = 6;
  const size_t smem = (size_t)STAGES * (128 * 64 * 2 + 128 * 64 * 2) + 1024;
  auto k = gemm_tc05_pair_kernel<STAGES, TO, EPI>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  const int pairs = tiles < si_sm_count() / 2 ? tiles : si_sm_count() / 2;
  if (pairs < 1) return -2;
  si_launch(k, dim3(2 * pairs), dim3(192), smem, stream, am, bm_half, (TO*)out, ldo, M, N, K, status);
  return si_last_error();
}

template <int STAGES, typename TO, int EPI>
static int launch(const CUtensorMap& am, const CUtensorMap& bm, void* out, long long ldo, int M, int N, int K,
                  int* status, cudaStream_t stream) {
  const size_t smem = (size_t)STAGES * (128 * 64 * 2 + 256 * 64 * 2) + 1024;
  auto k = gemm_tc05_kernel<STAGES, TO, EPI>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int tiles = ((M + 127) / 128) * ((N + 255) / 256);
  const int blocks = tiles < si_sm_count() ? tiles : si_sm_count();
  si_launch(k, dim3(blocks), dim3(192), smem, stream, am, bm, (TO*)out, ldo, M, N, K, status);
  return si_last_error();
}

// 1 when the driver can encode tensor maps (the kernel cannot run without TMA).
SI_EXPORT int si_gemm_tc05_ok() { return si_encode_fn() != nullptr; }

// The weight's tensor map (boxes of [256, 64]); made once per weight. `map_out`: 128 bytes, 64-byte aligned.
// `box_rows`: 256 for the one-CTA kernel, 128 for the kernel of CTA pairs (each CTA fetches half of the tile's rows).
SI_EXPORT int si_gemm_tc05_encode_weight(void* map_out, const void* W, int N, int K, long long ldw, int box_rows) {
  if ((K % 8) || (ldw % 8) || ((uintptr_t)W % 16) || (box_rows != 128 && box_rows != 256)) return -2;
  return si_encode_bf16_2d((CUtensorMap*)map_out, W, (unsigned long long)N, (unsigned long long)K,
                           (unsigned long long)ldw, (unsigned)box_rows);
}

// Products of more than 128 rows go to the kernel of CTA pairs when the caller has a map with boxes of 128 rows.
static bool use_pair(int M, const void* wmap_half) { return wmap_half && M > 128 && pair_enabled() && si_sm_count() >= 2; }

static int gemm_tc05_common(const void* x, long long ldx, const void* wmap, CUtensorMap* am, int M, int K) {
  if (K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)x % 16) || !wmap) return -2;
  return si_encode_bf16_2d(am, x, (unsigned long long)M, (unsigned long long)K, (unsigned long long)ldx, 128);
}

// out_dtype: SI_BF16 or SI_F32. x: [M, K] bf16 rows `ldx` apart. Returns -2 for unsupported sizes.
// `wmap`: the weight's map with boxes of 256 rows; `wmap_half` (may be null): the one with boxes of 128 rows.
SI_EXPORT int si_gemm_tc05(const void* x, long long ldx, const void* wmap, const void* wmap_half, void* out, long long ldo,
                           int out_dtype, int M, int N, int K, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  CUtensorMap am;
  const int rc = gemm_tc05_common(x, ldx, wmap, &am, M, K);
  if (rc) return rc;
  if (use_pair(M, wmap_half)) {
    const CUtensorMap& bh = *(const CUtensorMap*)wmap_half;
    if (out_dtype == SI_BF16) return launch_pair<bf16, EPI_STORE>(am, bh, out, ldo, M, N, K, status, stream);
    return launch_pair<float, EPI_STORE>(am, bh, out, ldo, M, N, K, status, stream);
  }
  const CUtensorMap& bm = *(const CUtensorMap*)wmap;
  if (out_dtype == SI_BF16) return launch<4, bf16, EPI_STORE>(am, bm, out, ldo, M, N, K, status, stream);
  return launch<4, float, EPI_STORE>(am, bm, out, ldo, M, N, K, status, stream);
}

// out[M, F] = silu(gate) * up (bf16) of the stacked projection x[M, K] W[2F, K]^T whose rows are interleaved in
// groups of 8 (8 gates, their 8 ups, ...); F a multiple of 8.
SI_EXPORT int si_gemm_tc05_swiglu(const void* x, long long ldx, const void* wmap, const void* wmap_half, void* out,
                                  long long ldo, int M, int F, int K, int* status, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return 0;
  if (F % 8) return -2;
  CUtensorMap am;
  const int rc = gemm_tc05_common(x, ldx, wmap, &am, M, K);
  if (rc) return rc;
  if (use_pair(M, wmap_half)) return launch_pair<bf16, EPI_SWIGLU>(am, *(const CUtensorMap*)wmap_half, out, ldo, M, 2 * F, K, status, stream);
  const CUtensorMap& bm = *(const CUtensorMap*)wmap;
  return launch<4, bf16, EPI_SWIGLU>(am, bm, out, ldo, M, 2 * F, K, status, stream);
}

// resid[M, N] (fp32, rows `ldr` apart) += x[M, K] W[N, K]^T, each sum rounded to bf16 before it is added: the
// output projection of a mixer or a feed-forward added into the residual stream by the product itself.
SI_EXPORT int si_gemm_tc05_add(const void* x, long long ldx, const void* wmap, const void* wmap_half, float* resid,
                               long long ldr, int M, int N, int K, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  CUtensorMap am;
  const int rc = gemm_tc05_common(x, ldx, wmap, &am, M, K);
  if (rc) return rc;
  if (use_pair(M, wmap_half)) return launch_pair<float, EPI_ADD>(am, *(const CUtensorMap*)wmap_half, resid, ldr, M, N, K, status, stream);
  return launch<4, float, EPI_ADD>(am, *(const CUtensorMap*)wmap, resid, ldr, M, N, K, status, stream);
}
