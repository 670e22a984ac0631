// Self-test of the bounded wait that every TMA-fed kernel of the package relies on: a wait on an mbarrier
// that nothing ever arrives at gives up after its limit, the kernel writes SI_WAIT_LIMIT into the status word
// and returns, and the host reads the word as after any step. Nothing traps, faults or spins on. The
// reference has no counterpart (its kernels have no waits; a failed step retires every request,
// src/source/scheduler/scheduler.cpp:496-513).
#include "tma_common.cuh"

__global__ void wait_runs_out_kernel(int* status, int limit, int* gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) mbar_init(&bar, 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool done = mbar_wait_limited(&bar, 0, limit);     // phase 0 never completes: no one arrives
    if (!done) set_status(status, SI_WAIT_LIMIT);
    if (gave_up) *gave_up = done ? 0 : 1;
  }
}

// `limit`: probes before the wait gives up (1 .. 2^20). Returns 0, a CUDA error code, or -2 (limit refused).
SI_EXPORT int si_selftest_wait_runs_out(int* status, int limit, int* gave_up, cudaStream_t stream) {
  if (limit < 1 || limit > (1 << 20)) return -2;
  wait_runs_out_kernel<<<1, 32, 0, stream>>>(status, limit, gave_up);
  return si_last_error();
}
