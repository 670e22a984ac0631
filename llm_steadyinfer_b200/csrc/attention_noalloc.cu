// Split decode attention with library-owned scratch: see attention_noalloc.h for who needs
// this and the rules. The kernel is the cp.async decode kernel of attention_mma.cu, compiled
// into this library again by including that file; only where its scratch comes from differs.
#define SI_EXPORT extern "C" __attribute__((visibility("hidden")))   // attention_mma.cu's entry points stay in its own library
#include "attention_noalloc.h"
#include "attention_mma.cu"
#include <atomic>
#include <stdio.h>

// The scratch itself: tickets first (a fixed region, so their place never depends on a
// call's sizes), partial results behind them. Device code may name this array; host code
// may not use the name as an address and asks the runtime for it instead.
static __device__ __align__(256) float g_noalloc_scratch[SI_NOALLOC_MAX_UNITS + SI_NOALLOC_SCRATCH_WORDS];

#define SI_NOALLOC_MAX_DEVICES 64
static std::atomic<float*> g_scratch_addr[SI_NOALLOC_MAX_DEVICES];      // device address per device, once looked up
static thread_local char g_error[256] = "";

extern "C" __attribute__((visibility("default"))) const char* si_noalloc_last_error(void) { return g_error; }

extern "C" __attribute__((visibility("default")))
long long si_attn_decode_noalloc_words(int num_items, int H, int KV, int hs, int nsplit) {
  if (KV <= 0 || H % KV) return -1;
  const long long rows = si_attn_decode_rows(H, KV, hs);
  if (rows <= 0) return -1;
  if (nsplit <= 1) return 0;
  return (long long)num_items * KV * nsplit * rows * (hs + 2);
}

template <int HS_PAD, int MT>
static bool decode_smem_limit() {
  return set_smem(attn_decode_kernel<HS_PAD, MT, decode_stages<HS_PAD>()>, decode_smem_bytes<HS_PAD, MT>()) == 0;
}
// Every variant that si_attn_decode_noalloc may launch; touching them also loads the module on the device.
static bool set_decode_smem_limits() {
  return decode_smem_limit<64, 1>() && decode_smem_limit<64, 2>() && decode_smem_limit<64, 4>() &&
         decode_smem_limit<128, 1>() && decode_smem_limit<128, 2>() && decode_smem_limit<256, 1>();
}

// Device address of the scratch array on the current device; looked up on the first call.
static int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= SI_NOALLOC_MAX_DEVICES) {
    snprintf(g_error, sizeof g_error, "cannot identify the current device (%s)", cudaGetErrorString(e));
    return SI_NOALLOC_SETUP_FAILED;
  }
  float* ptr = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (!ptr) {
    // Threads that get here together each ask the runtime; it gives them all the same address.
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      snprintf(g_error, sizeof g_error, "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      return SI_NOALLOC_SETUP_FAILED;
    }
    if (!set_decode_smem_limits()) {
      snprintf(g_error, sizeof g_error, "setting the kernels' shared-memory limits failed on device %d", dev);
      return SI_NOALLOC_SETUP_FAILED;
    }
    g_scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return 0;
}

extern "C" __attribute__((visibility("default"))) int si_noalloc_init(void) {
  g_error[0] = 0;
  float* base = nullptr;
  return scratch_for_current_device(&base);
}

extern "C" __attribute__((visibility("default"))) int si_noalloc_poison_tickets(int units, cudaStream_t stream) {
  g_error[0] = 0;
  if (units < 0 || units > SI_NOALLOC_MAX_UNITS) return -2;
  float* base = nullptr;
  const int rc = scratch_for_current_device(&base);
  if (rc) return rc;
  return (int)cudaMemsetAsync(base, 0x5a, (size_t)units * sizeof(int), stream);
}

extern "C" __attribute__((visibility("default")))
int si_attn_decode_noalloc(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                           const int* block_table, int table_width, const void* items, int num_items,
                           void* out, long long out_stride, int num_pages, int page_size, int num_seqs,
                           int H, int KV, int hs, float scale, int window, int nsplit, int* status,
                           cudaStream_t stream) {
  g_error[0] = 0;
  if (num_items <= 0) return 0;
  AttnParams p;
  if (!fill_params(p, q, q_stride, k_cache, v_cache, block_table, table_width, items, out, out_stride, num_pages,
                   page_size, num_seqs, H, KV, hs, scale, window, status)) {
    snprintf(g_error, sizeof g_error, "head layout or strides not supported (H=%d KV=%d head_dim=%d)", H, KV, hs);
    return -2;
  }
  const int rows = si_attn_decode_rows(H, KV, hs);
  if (rows <= 0 || nsplit < 1 || nsplit > 65535) {
    snprintf(g_error, sizeof g_error, "%d query heads per kv head or %d splits are outside the kernel's range", H / KV, nsplit);
    return -2;
  }
  p.nsplit = nsplit;
  if (nsplit > 1) {
    const long long words = si_attn_decode_noalloc_words(num_items, H, KV, hs, nsplit);
    const long long units = (long long)num_items * KV;
    if (words > SI_NOALLOC_SCRATCH_WORDS || units > SI_NOALLOC_MAX_UNITS) {
      snprintf(g_error, sizeof g_error,
               "scratch needed: %lld words and %lld tickets; the fixed array holds %d words and %d tickets",
               words, units, SI_NOALLOC_SCRATCH_WORDS, SI_NOALLOC_MAX_UNITS);
      return SI_NOALLOC_TOO_LARGE;
    }
    float* base = nullptr;
    const int rc = scratch_for_current_device(&base);
    if (rc) return rc;
    p.counters = reinterpret_cast<int*>(base);
    p.part_o = base + SI_NOALLOC_MAX_UNITS;
    p.part_ml = p.part_o + (size_t)num_items * KV * nsplit * rows * hs;
    // the tickets must start at zero whatever an earlier call (or an aborted one) left there
    cudaError_t e = cudaMemsetAsync(p.counters, 0, (size_t)units * sizeof(int), stream);
    if (e != cudaSuccess) {
      snprintf(g_error, sizeof g_error, "clearing the tickets failed: %s", cudaGetErrorString(e));
      return (int)e;
    }
  }
  if (hs <= 64) {
    if (rows == 16) return launch_decode<64, 1>(p, num_items, stream);
    if (rows == 32) return launch_decode<64, 2>(p, num_items, stream);
    return launch_decode<64, 4>(p, num_items, stream);
  }
  if (hs <= 128) {
    if (rows == 16) return launch_decode<128, 1>(p, num_items, stream);
    return launch_decode<128, 2>(p, num_items, stream);
  }
  return launch_decode<256, 1>(p, num_items, stream);
}
