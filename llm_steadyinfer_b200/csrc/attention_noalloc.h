/* Decode attention for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference project; it exists for hosts that
 * embed the kernels where device allocation is off limits at call time: code that runs
 * inside a memory-pool-managed runtime which forbids cudaMalloc after start-up, plug-ins
 * loaded into another process's CUDA context with a fixed memory budget, and real-time
 * loops in which an allocation (a device-wide synchronising call) would break the latency
 * bound. Such callers still own the inputs and outputs; only the kernel's scratch memory
 * (the per-split partial results and the merge tickets of split decode attention) is
 * provided by the library, from a fixed array that lives in the loaded module.
 *
 * Limits and rules
 *  - The scratch array holds SI_NOALLOC_SCRATCH_WORDS 4-byte words (16 MiB, plus 256 KiB of
 *    tickets) on every device that loads the library's device code, until the process exits. With
 *    the CUDA runtime's lazy module loading that is not the moment the shared library is opened but
 *    the first use of the module on a device: si_noalloc_init(), or failing that the first call of
 *    si_attn_decode_noalloc(). That first use is where the driver reserves the array (an allocation
 *    by the driver, not by this code): it can fail or stall for a caller with a fixed memory budget,
 *    so make it at start-up, outside any window in which nothing may be allocated. A call needs
 *      num_items * KV * nsplit * rows * (head_dim + 2) words,  rows = 16, 32 or 64
 *    (si_attn_decode_noalloc_words() computes it) and at most SI_NOALLOC_MAX_UNITS
 *    (num_items * KV) tickets; larger requests are refused with SI_NOALLOC_TOO_LARGE and
 *    nothing is launched. si_noalloc_last_error() gives the reason in words.
 *  - si_noalloc_init(), with the device current, loads the module there, looks up the array's
 *    device address (cudaGetSymbolAddress) and sets the kernels' shared-memory limits. Call it once
 *    per device at start-up. If it was not called, the first si_attn_decode_noalloc() on a device
 *    does the same work: then make that first call outside any stream capture and outside any
 *    no-allocation window. Both may be called from several host threads.
 *  - The address is remembered per device ordinal, that is for the device's primary context, which
 *    the runtime API uses. A host that makes other contexts current on the same device (driver API)
 *    must not call this entry point in them: the remembered address is valid in the primary one only.
 *  - All calls share the one array, and it keeps what the last call left. The ticket words
 *    are cleared by every call before its kernel runs; partial results are overwritten
 *    before they are read. Two calls whose kernels overlap on the GPU (different streams
 *    without an ordering between them) race on the array: order them.
 *  - This code calls no cudaMalloc, cudaFree or other allocating routine on any path; what the
 *    driver reserves when the module is first used on a device is described above.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SI_NOALLOC_SCRATCH_WORDS (4 * 1024 * 1024)
#define SI_NOALLOC_MAX_UNITS 65536
#define SI_NOALLOC_TOO_LARGE (-4)
#define SI_NOALLOC_SETUP_FAILED (-5)

/* Same arguments and result codes as si_attn_decode (attention_mma.cu) without the scratch
 * pointer: q [T, H*hs] bf16 rows (row stride in elements), one layer's K and V cache
 * [num_pages, KV, page_size, hs] bf16, the step's block table, work items (sequence, first
 * row, tokens, first position), output rows, and the number of splits of the key range. */
int si_attn_decode_noalloc(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                           const int* block_table, int table_width, const void* items, int num_items,
                           void* out, long long out_stride, int num_pages, int page_size, int num_seqs,
                           int H, int KV, int hs, float scale, int window, int nsplit, int* status,
                           cudaStream_t stream);

/* Set-up for the current device (see the rules above): 0, or SI_NOALLOC_SETUP_FAILED with the reason in
 * si_noalloc_last_error(). Cheap when the device is set up already. */
int si_noalloc_init(void);

/* Words of scratch a call with these sizes needs (0 when nsplit is 1), or -1 for a head
 * layout the kernel does not take. */
long long si_attn_decode_noalloc_words(int num_items, int H, int KV, int hs, int nsplit);

/* For tests of this entry point: fills the first `units` ticket words with a non-zero pattern on `stream`,
 * as a call that was cut short might leave them. Every call clears the tickets it uses before its kernel
 * runs, so a following call must be unaffected. Returns 0 or an error code. */
int si_noalloc_poison_tickets(int units, cudaStream_t stream);

/* Text of the last refusal or set-up failure on the calling thread ("" if none). */
const char* si_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
