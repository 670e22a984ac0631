// Shared device helpers for every kernel file: element load/store through fp32,
// warp and block reductions, and the status word that kernels write instead of
// trapping. Each .cu file is compiled on its own into one shared library and
// exports plain C entry points that take raw device pointers and a stream.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

// A file that includes another .cu file to reuse its kernels defines SI_EXPORT first (hidden visibility),
// so that the included file's entry points are not exported a second time from its library.
#ifndef SI_EXPORT
#define SI_EXPORT extern "C" __attribute__((visibility("default")))
#endif

// Status codes written (atomicMax) into the engine's device status word.
enum SiStatus : int {
  SI_OK = 0,
  SI_BAD_TOKEN = 1,      // token id outside [0, vocab)
  SI_BAD_PAGE = 2,       // block table entry outside [0, num_pages)
  SI_BAD_SEQ = 3,        // row names a sequence outside the batch
  SI_WAIT_LIMIT = 4,     // a bounded wait inside a kernel ran out
};

// dtype codes shared with the Python binding
enum SiDtype : int { SI_F32 = 0, SI_BF16 = 1 };

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();                 // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float s = lane < nwarps ? scratch[lane] : 0.f;
    s = warp_sum(s);
    if (lane == 0) scratch[32] = s;
  }
  __syncthreads();
  return scratch[32];
}

// The feed-forward's gated activation: silu(g) * u in fp32.
__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.f + expf(-g))) * u; }

__device__ __forceinline__ void set_status(int* status, int code) {
  if (status) atomicMax(status, code);
}

// Programmatic dependent launch: a kernel that starts with pdl_prologue() lets the next kernel of
// the stream begin launching while it still runs, and itself waits for the previous kernel's
// results before touching any memory. Launched through si_launch() the kernel carries the
// attribute that allows this overlap of launch latency; launched with <<<>>> both instructions
// do nothing. SI_PDL=0 in the environment turns the attribute off.
__device__ __forceinline__ void pdl_prologue() {
#ifdef SI_PDL_EARLY_TRIGGER
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
#endif
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

// A hint that [base, base + bytes) will be streamed soon: block `part` of `parts` asks the memory system
// to bring its share into L2, one prefetch per 128-byte line. Kernels that wait on latency while HBM
// idles (the norms of a decode step) call this for the first weights of the matrix product after them.
__device__ __forceinline__ void l2_prefetch_share(const void* base, long long bytes, int part, int parts) {
  constexpr long long LINE = 128;
  const long long lines = bytes / LINE;
  const long long per = (lines + parts - 1) / parts;
  const long long c0 = (long long)part * per;
  const long long c1 = c0 + per < lines ? c0 + per : lines;
  for (long long c = c0 + threadIdx.x; c < c1; c += blockDim.x)
    asm volatile("prefetch.global.L2 [%0];\n" :: "l"(reinterpret_cast<const char*>(base) + c * LINE) : "memory");
}

// The two halves of pdl_prologue() for kernels that place them themselves. A small kernel (a norm, the
// position encoding) calls pdl_trigger() at its start: the kernel after it may then become resident and do
// whatever does not depend on this one (set-up, the first loads of its weights) before its own pdl_wait().
// Kernels of more than one wave do not trigger: blocks of the next kernel that sit waiting would take the
// places of their own later blocks.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// SI_PDL_TRIGGER: 0 no kernel triggers; 1 the small kernels; 2 (default) also every kernel of one wave of
// blocks, at its start; 3 also kernels of several waves, once their main loop is done.
static inline int si_pdl_trigger_level() {
  static int level = -1;
  if (level < 0) {
    const char* e = getenv("SI_PDL_TRIGGER");
    level = (e && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 2;
  }
  return level;
}
static inline bool si_pdl_trigger_enabled() { return si_pdl_trigger_level() >= 1; }
// What a kernel of `blocks` blocks, `slots` of which run at once, is told: 0 do not trigger, 1 at the
// start, 2 after the main loop.
static inline int si_pdl_trigger_mode(long long blocks, long long slots) {
  const int level = si_pdl_trigger_level();
  if (blocks <= slots) return level >= 2 ? 1 : 0;
  return level >= 3 ? 2 : 0;
}

// Streaming multiprocessors of the current device, asked once per device. Grid sizes that should fill the
// device once ("one wave") are derived from it; no kernel's result depends on it.
static inline int si_sm_count() {
  static int count[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    count[dev] = n;
  }
  return count[dev];
}

static inline bool si_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("SI_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

template <typename... P, typename... A>
static inline void si_launch(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = si_pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, P(args)...);
}

static inline int si_last_error() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}
