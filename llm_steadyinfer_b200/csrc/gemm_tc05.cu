// bf16 matrix product on the 5th-generation tensor cores: out[M, N] = x[M, K] * W[N, K]^T with
// fp32 accumulation in tensor memory. The reference leaves every product to cuBLAS
// (src/source/op/kernels/cuda/matmul_kernel.cu:128-150); this is the package's own kernel for
// products with many rows (prompt portions).
//
// One block computes a 128 x BN tile. Warp 0 is the TMA producer: per 64-wide k step it fetches a
// [128, 64] box of x and a [BN, 64] box of W (128-byte swizzle) into a ring of stages. Warp 1
// issues tcgen05.mma (four K=16 instructions per stage, descriptors advanced by 32 bytes) into the
// tensor-memory accumulator and releases each stage with tcgen05.commit. Warps 2-5 wait for the
// last commit, read their 32 accumulator lanes with tcgen05.ld and store the rows. All waits are
// bounded; a wait that runs out sets SI_WAIT_LIMIT and the block leaves without storing.
#include "tma_common.cuh"

typedef __nv_bfloat16 bf16;

template <typename TO> __device__ __forceinline__ void store_row32(TO* dst, const float (&v)[32], int valid, bool vec);
template <> __device__ __forceinline__ void store_row32<float>(float* dst, const float (&v)[32], int valid, bool vec) {
  if (vec && valid == 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
    for (int i = 0; i < valid; ++i) dst[i] = v[i];
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
    for (int i = 0; i < valid; ++i) dst[i] = __float2bfloat16_rn(v[i]);
  }
}

template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(192)
gemm_tc05_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
                 TO* __restrict__ out, long long ldo, int M, int N, int K, int* status) {
  constexpr int BM = 128, BK = 64;
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ unsigned tmem_slot;
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* As = smem;
  unsigned char* Bs = smem + STAGES * A_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int nk = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, BN);
  tc05_fence_before_sync();
  __syncthreads();
  tc05_fence_after_sync();
  const unsigned tmem = tmem_slot;

  if (warp == 0 && lane == 0) {
    for (int kb = 0; kb < nk; ++kb) {
      const int s = kb % STAGES;
      if (kb >= STAGES && !mbar_wait(&empty_bar[s], (unsigned)(((kb / STAGES) - 1) & 1))) {
        set_status(status, SI_WAIT_LIMIT);
        break;
      }
      mbar_expect_tx(&full_bar[s], A_BYTES + B_BYTES);
      tma_load_2d(As + s * A_BYTES, &amap, &full_bar[s], kb * BK, m0);
      tma_load_2d(Bs + s * B_BYTES, &bmap, &full_bar[s], kb * BK, n0);
    }
  } else if (warp == 1 && lane == 0) {
    constexpr unsigned idesc = umma_idesc_bf16(BM, BN, false);
    bool ok = true;
    for (int kb = 0; kb < nk && ok; ++kb) {
      const int s = kb % STAGES;
      ok = mbar_wait(&full_bar[s], (unsigned)((kb / STAGES) & 1));
      if (!ok) { set_status(status, SI_WAIT_LIMIT); break; }
      tc05_fence_after_sync();
      const unsigned long long ad = umma_desc_sw128(As + s * A_BYTES, 16, 1024);
      const unsigned long long bd = umma_desc_sw128(Bs + s * B_BYTES, 16, 1024);
#pragma unroll
      for (int k = 0; k < BK / 16; ++k)
        tc05_mma_bf16(tmem, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
      tc05_commit(&empty_bar[s]);            // the stage is free once these instructions have read it
    }
    tc05_commit(&acc_bar);                    // the accumulator is complete
  } else if (warp >= 2) {
    const int q = warp & 3;                   // the 32 tensor-memory lanes this warp may read
    const bool ok = mbar_wait(&acc_bar, 0);
    if (!__all_sync(0xffffffffu, ok)) {
      if (lane == 0) set_status(status, SI_WAIT_LIMIT);
    } else {
      tc05_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const bool vec = (ldo % 8 == 0) && ((uintptr_t)out % 16 == 0);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float v[32];
        tmem_ld_32x32(tmem + ((unsigned)(q * 32) << 16) + (unsigned)(c * 32), v);
        const int n = n0 + c * 32;
        if (row < M && n < N) store_row32<TO>(out + (size_t)row * ldo + n, v, min(32, N - n), vec);
      }
    }
  }
  tc05_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, BN);
}

template <int BN, int STAGES, typename TO>
static int launch(const CUtensorMap& am, const CUtensorMap& bm, void* out, long long ldo, int M, int N, int K,
                  int* status, cudaStream_t stream) {
  const size_t smem = (size_t)STAGES * (128 * 64 * 2 + BN * 64 * 2) + 1024;
  auto k = gemm_tc05_kernel<BN, STAGES, TO>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((N + BN - 1) / BN, (M + 127) / 128);
  k<<<grid, 192, smem, stream>>>(am, bm, (TO*)out, ldo, M, N, K, status);
  return si_last_error();
}

// 1 when the driver can encode tensor maps (the kernel cannot run without TMA).
SI_EXPORT int si_gemm_tc05_ok() { return si_encode_fn() != nullptr; }

// The weight's tensor map (boxes of [128, 64]); made once per weight. `map_out`: 128 bytes, 64-byte aligned.
SI_EXPORT int si_gemm_tc05_encode_weight(void* map_out, const void* W, int N, int K, long long ldw) {
  if ((K % 8) || (ldw % 8) || ((uintptr_t)W % 16)) return -2;
  return si_encode_bf16_2d((CUtensorMap*)map_out, W, (unsigned long long)N, (unsigned long long)K,
                           (unsigned long long)ldw, 128);
}

// out_dtype: SI_BF16 or SI_F32. x: [M, K] bf16 rows `ldx` apart. Returns -2 for unsupported sizes.
SI_EXPORT int si_gemm_tc05(const void* x, long long ldx, const void* wmap, void* out, long long ldo, int out_dtype,
                           int M, int N, int K, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)x % 16) || !wmap) return -2;
  CUtensorMap am;
  const int rc = si_encode_bf16_2d(&am, x, (unsigned long long)M, (unsigned long long)K, (unsigned long long)ldx, 128);
  if (rc) return rc;
  const CUtensorMap& bm = *(const CUtensorMap*)wmap;
  if (out_dtype == SI_BF16) return launch<128, 6, bf16>(am, bm, out, ldo, M, N, K, status, stream);
  return launch<128, 6, float>(am, bm, out, ldo, M, N, K, status, stream);
}
