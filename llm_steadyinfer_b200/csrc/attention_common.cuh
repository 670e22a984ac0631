// Shared by the attention kernels: the work item and parameter structs and thin wrappers of
// the PTX instructions they use (cp.async, ldmatrix, mma.sync m16n8k16 bf16).
#pragma once
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

struct AttnItem { int seq, row0, ntok, pos0; };

// The split decode kernels keep one ticket per (item, kv head) at the START of their scratch, in a
// region of this fixed size that never holds anything else: the scratch is shared by launches with
// different numbers of items and splits, and a ticket that lay behind the partial results would
// fall, after such a change, on a word that an earlier launch has left a partial result in.
#define SI_ATTN_TICKETS 65536

// The first key that any row of an item can see: with a window of w keys the item's first token, at
// position pos0, reads keys pos0 - w + 1 onwards. Keys before it are never fetched and their pages
// never looked up: the cache manager has given those pages back, and their table entries say so.
__device__ __forceinline__ int window_first_key(int pos0, int window) {
  return window > 0 && pos0 - window + 1 > 0 ? pos0 - window + 1 : 0;
}

struct AttnParams {
  const bf16* q; long long q_stride;
  const bf16* k_cache; const bf16* v_cache;
  const int* block_table; int table_width;
  const AttnItem* items;
  bf16* out; long long out_stride;
  float* part_o;            // [item][kv head][split][row][hs]  (decode kernel with nsplit > 1)
  float* part_ml;           // [item][kv head][split][row][2]
  int* counters;            // [item][kv head] tickets of the split merge, zero between launches
  int num_pages, page_size, num_seqs, H, KV, G, hs;
  float scale_log2;         // scale * log2(e)
  int window, nsplit;
  int* status;
};

// ---- small PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;       // src-size 0 zero-fills the 16 bytes
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 2^x in fp32 by the hardware approximation (2 ulp); exp2(-inf) = 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

