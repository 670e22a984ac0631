// TMA, mbarrier and tcgen05 helpers shared by the kernels that use them: thin wrappers of the
// PTX instructions, every wait bounded, and the host-side encoding of 2-D bf16 tensor maps.
#pragma once
#include "common.cuh"
#include <cuda.h>
#include <stdint.h>

__device__ __forceinline__ unsigned tma_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tma_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tma_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(tma_smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tma_smem_u32(bar)) : "memory");
}
// Bounded wait: false when the phase did not complete within `limit` further probes.
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, unsigned parity, int limit) {
  if (mbar_try_wait(bar, parity)) return true;       // the common case costs one probe, not a loop
  for (int it = 0; it < limit; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// The limit every kernel of the package waits with (tens of milliseconds; a tile arrives in microseconds).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
  return mbar_wait_limited(bar, parity, 1 << 20);
}
// The same wait for a whole warp: after one probe by all lanes, one lane polls and the others get
// its answer.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, unsigned parity) {
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;   // already complete: one probe by all
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(tma_smem_u32(dst)), "l"(map), "r"(tma_smem_u32(bar)), "r"(x), "r"(y) : "memory");
}


// ---- tcgen05 (5th generation tensor cores, accumulators in tensor memory) ------------------------
// Allocate `ncols` (power of two >= 32) columns of tensor memory; executed by one whole warp.
// The base address lands in shared memory at `slot`.
__device__ __forceinline__ void tmem_alloc(unsigned* slot, unsigned ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tma_smem_u32(slot)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc05_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc05_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// True in exactly one lane of a converged warp. The tensor-core instructions take their operands from
// warp-uniform values: code that the whole warp runs, with only the instruction itself under this
// predicate, lets the compiler keep descriptors and addresses in uniform registers, which a branch
// on the lane number does not.
__device__ __forceinline__ bool elect_one() {
  unsigned pred;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues.
__device__ __forceinline__ void tc05_mma_bf16(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                              unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// The mbarrier gets one arrival when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tma_smem_u32(bar)) : "memory");
}
// 32 lanes x 32 columns of fp32 from tensor memory: thread i of the warp gets lane (base + i).
__device__ __forceinline__ void tmem_ld_32x32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The same without the wait: several loads can be in flight before one tmem_ld_wait().
__device__ __forceinline__ void tmem_ld_32x32_issue(unsigned taddr, float* v) {
  unsigned* r = reinterpret_cast<unsigned*>(v);
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// 32 lanes x 32 columns of fp32 into tensor memory, then wait for the store.
__device__ __forceinline__ void tmem_st_32x32(unsigned taddr, const float (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
               :: "r"(taddr),
                  "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                  "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                  "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                  "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                  "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                  "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                  "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                  "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
               : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// 32 lanes x 32 columns of raw 32-bit words into tensor memory without waiting; tmem_st_wait() after the
// last one. Packed bf16 pairs written this way form the A operand of tc05_mma_bf16_tmem_a.
__device__ __forceinline__ void tmem_st_32x32_issue(unsigned taddr, const unsigned* v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
               "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
               :: "r"(taddr),
                  "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                  "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
                  "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                  "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem desc]: A is 128 rows (tensor-memory lanes) x 16 bf16, two to a 32-bit
// column (element 2c in the low half of column c), so one step reads 8 columns from `a_tmem`.
__device__ __forceinline__ void tc05_mma_bf16_tmem_a(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc,
                                                     unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// ---- pairs of CTAs on one tile (tcgen05 with cta_group::2) ----------------------------------------
// The two CTAs of a cluster of two take one 256-row tile together: each holds 128 rows of A, half of the rows
// of B and its 128 rows of the accumulator; CTA 0 (the leader) issues the instructions, which read both CTAs'
// shared memory at equal offsets. Every helper below is for such a pair.
__device__ __forceinline__ unsigned cluster_cta_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The shared::cluster address of `p` (a shared-memory object of this CTA) as CTA `rank` of the cluster holds it.
__device__ __forceinline__ unsigned cluster_map_u32(const void* p, unsigned rank) {
  unsigned a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(a) : "r"(tma_smem_u32(p)), "r"(rank));
  return a;
}
// One arrival at an mbarrier given by its shared::cluster address (this CTA's or the peer's).
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose bytes are counted at an mbarrier of either CTA of the pair
// (`bar_cluster_addr`: shared::cluster address). No multicast: each CTA fetches its own boxes.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, unsigned bar_cluster_addr, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(tma_smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
// Tensor memory of both CTAs of the pair; one warp of each CTA runs this.
__device__ __forceinline__ void tmem_alloc_pair(unsigned* slot, unsigned ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tma_smem_u32(slot)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(unsigned taddr, unsigned ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B over the pair's 256 rows; issued by one thread of the leader CTA.
__device__ __forceinline__ void tc05_mma_bf16_pair(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                                   unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// One arrival at the mbarrier at this offset in each CTA of `cta_mask` once every tcgen05.mma issued so far
// by this thread has completed. (A multicast of an arrival, not of a load.)
__device__ __forceinline__ void tc05_commit_pair(uint64_t* bar, unsigned short cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
               ::"r"(tma_smem_u32(bar)), "h"(cta_mask) : "memory");
}

// Shared-memory matrix descriptor of a bf16 tile whose rows are 128 bytes (64 elements) apart and
// swizzled in 8-row, 1024-byte groups (the 128-byte TMA swizzle); the tile must start on a 1024-byte
// boundary. K-major operand (rows = M or N, the 64 columns = K): groups of 8 rows lie `sbo` bytes apart.
// MN-major operand (rows = K, the 64 columns = M or N): groups of 8 k-rows lie `sbo` bytes apart and the
// next 64 columns start `lbo` bytes further.
__device__ __forceinline__ unsigned long long umma_desc_sw128(const void* smem, unsigned lbo, unsigned sbo) {
  unsigned long long d = 0;
  d |= (unsigned long long)((tma_smem_u32(smem) >> 4) & 0x3fff);
  d |= (unsigned long long)((lbo >> 4) & 0x3fff) << 16;
  d |= (unsigned long long)((sbo >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;                 // descriptor version of this architecture
  d |= 2ull << 61;                 // 128-byte swizzle
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, M x N tile, A K-major; B K-major or MN-major.
__host__ __device__ constexpr unsigned umma_idesc_bf16(int M, int N, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((unsigned)(N >> 3) << 17) |
         ((unsigned)(M >> 4) << 24);
}

// ---- host: tensor maps --------------------------------------------------------------------------
typedef CUresult (*SiEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline SiEncodeTiledFn si_encode_fn() {
  static SiEncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (SiEncodeTiledFn)ptr;
  }
  return fn;
}

// bf16 matrix [rows, cols] with `row_stride` elements between rows, boxes of [box_rows, 64 columns],
// 128-byte swizzle. Returns 0, -3 (no driver entry point) or 1000 + the driver's error code.
static inline int si_encode_bf16_2d(CUtensorMap* map, const void* base, unsigned long long rows,
                                    unsigned long long cols, unsigned long long row_stride, unsigned box_rows) {
  SiEncodeTiledFn fn = si_encode_fn();
  if (!fn) return -3;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}
