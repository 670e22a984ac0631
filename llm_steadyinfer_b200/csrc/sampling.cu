// Token selection from fp32 logits: one block per row (sample_kernel), or, for batches that are greedy
// throughout, the vocabulary of a row split over 32 blocks (argmax_split_kernel).
//  * greedy: argmax, ties to the lowest index, as the reference's batch argmax
//    (src/source/op/kernels/cuda/argmax_kernel.cu:14-19, 93-117).
//  * temperature / top-k / top-p: p_i = exp((x_i - max) / T); keep the k largest logits
//    (all ties of the k-th kept), then the smallest set of largest logits whose mass reaches
//    top_p of what top-k kept (ties kept); draw by inverse CDF in index order with a uniform
//    from a counter-based generator keyed by (seed, index of the output token), so that a
//    request regenerates the same tokens after preemption. The reference samples greedily only.
// The thresholds are found by bisection over the order-preserving integer image of the
// logits, so no sort and no scratch memory is needed.
#include "common.cuh"
#include <math.h>

#define SAMPLE_THREADS 1024

// Larger float, larger key; -0.0 and +0.0, equal as numbers, get the same key (they must tie like other equals).
__device__ __forceinline__ unsigned ordered_key(float x) {
  unsigned u = __float_as_uint(x);
  if (u == 0x80000000u) u = 0u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float block_reduce_sum_f(float v, float* sh) {
  return block_sum(v, sh);
}

__device__ __forceinline__ float block_reduce_max_f(float v, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float s = lane < nw ? sh[lane] : -INFINITY;
    s = warp_max(s);
    if (lane == 0) sh[32] = s;
  }
  __syncthreads();
  return sh[32];
}

// splitmix64 finaliser over (seed, counter) -> uniform in [0, 1) with 24 bits
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long counter) {
  unsigned long long z = seed ^ (counter * 0x9E3779B97F4A7C15ull);
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
              const unsigned long long* __restrict__ counter, int* __restrict__ out) {
  __shared__ float sh[33];
  __shared__ float chunk_sum[SAMPLE_THREADS];
  __shared__ int s_idx;
  pdl_prologue();
  const int r = blockIdx.x;
  const float* x = logits + (size_t)r * row_stride;
  const int tid = threadIdx.x;

  // row maximum and its lowest index
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = x[i];
    if (v > best) { best = v; best_i = i; }
  }
  const float mx = block_reduce_max_f(best, sh);
  if (tid == 0) s_idx = 0x7fffffff;
  __syncthreads();
  if (best == mx && best_i != 0x7fffffff) atomicMin(&s_idx, best_i);
  __syncthreads();
  const float T = temperature ? temperature[r] : 0.f;
  if (!(T > 0.f)) {
    if (tid == 0) out[r] = s_idx == 0x7fffffff ? 0 : s_idx;
    return;
  }
  const float invT = 1.f / T;
  const int k = top_k ? top_k[r] : 0;
  const float pp = top_p ? top_p[r] : 1.f;

  unsigned lo_key = 0;                       // keep logits whose key >= lo_key
  if (k > 0 && k < vocab) {
    // largest key u with count{key >= u} >= k
    unsigned lo = 0, hi = 0xffffffffu;
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1) + 1;
      float c = 0.f;
      for (int i = tid; i < vocab; i += blockDim.x) c += ordered_key(x[i]) >= mid ? 1.f : 0.f;
      c = block_reduce_sum_f(c, sh);
      if (c >= (float)k) lo = mid; else hi = mid - 1;
    }
    lo_key = lo;
  }
  // mass kept by top-k
  float z = 0.f;
  for (int i = tid; i < vocab; i += blockDim.x)
    if (ordered_key(x[i]) >= lo_key) z += expf((x[i] - mx) * invT);
  z = block_reduce_sum_f(z, sh);
  if (pp < 1.f) {
    const float target = pp * z;
    unsigned lo = lo_key, hi = ordered_key(mx);
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1) + 1;
      float s = 0.f;
      for (int i = tid; i < vocab; i += blockDim.x)
        if (ordered_key(x[i]) >= mid) s += expf((x[i] - mx) * invT);
      s = block_reduce_sum_f(s, sh);
      if (s >= target) lo = mid; else hi = mid - 1;
    }
    lo_key = lo;
    z = 0.f;
    for (int i = tid; i < vocab; i += blockDim.x)
      if (ordered_key(x[i]) >= lo_key) z += expf((x[i] - mx) * invT);
    z = block_reduce_sum_f(z, sh);
  }
  // inverse CDF in index order: thread i owns the contiguous chunk [i*c, (i+1)*c)
  const float u = uniform01(seed ? seed[r] : 0ull, counter ? counter[r] : 0ull);
  const float target = u * z;
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int b = tid * chunk, e = min(vocab, b + chunk);
  float mine = 0.f;
  for (int i = b; i < e; ++i)
    if (ordered_key(x[i]) >= lo_key) mine += expf((x[i] - mx) * invT);
  chunk_sum[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    // the walk over per-thread sums is short (1024 entries) and keeps one summation order
    float run = 0.f;
    int owner = -1;
    float before = 0.f;
    int last_nonempty = -1;
    for (int i = 0; i < (int)blockDim.x; ++i) {
      if (chunk_sum[i] > 0.f) last_nonempty = i;
      if (owner < 0 && chunk_sum[i] > 0.f && run + chunk_sum[i] > target) { owner = i; before = run; }
      run += chunk_sum[i];
    }
    if (owner < 0) { owner = last_nonempty; before = run - chunk_sum[owner < 0 ? 0 : owner]; }
    s_idx = owner;
    sh[0] = before;
  }
  __syncthreads();
  if (tid == s_idx) {
    float run = sh[0];
    int pick = -1, last = -1;
    for (int i = b; i < e; ++i) {
      if (ordered_key(x[i]) >= lo_key) {
        last = i;
        run += expf((x[i] - mx) * invT);
        if (run > target) { pick = i; break; }
      }
    }
    out[r] = pick >= 0 ? pick : last;
  }
}

// Greedy rows only: the vocabulary of a row is split over ARGMAX_SPLITS blocks, each leaves its
// (maximum, lowest index) in `scratch`, and the block that comes last (a ticket per row) merges them;
// it also puts the ticket back to zero for the next launch. One block per row, as in sample_kernel,
// leaves most of the SMs idle while a few of them read the whole row.
#define ARGMAX_SPLITS 32
#define ARGMAX_THREADS 256

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_split_kernel(const float* __restrict__ logits, long long row_stride, int vocab, float* __restrict__ part_max,
                    int* __restrict__ part_idx, int* __restrict__ tickets, int* __restrict__ out) {
  __shared__ float sh[33];
  __shared__ int s_idx, s_last;
  pdl_prologue();
  const int r = blockIdx.y, sp = blockIdx.x;
  const float* x = logits + (size_t)r * row_stride;
  const int per = (vocab + ARGMAX_SPLITS - 1) / ARGMAX_SPLITS;
  const int b = sp * per, e = min(vocab, b + per);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = b + threadIdx.x; i < e; i += ARGMAX_THREADS) {
    const float v = x[i];
    if (v > best) { best = v; best_i = i; }
  }
  const float mx = block_reduce_max_f(best, sh);
  if (threadIdx.x == 0) s_idx = 0x7fffffff;
  __syncthreads();
  if (best == mx && best_i != 0x7fffffff) atomicMin(&s_idx, best_i);
  __syncthreads();
  if (threadIdx.x == 0) {
    part_max[r * ARGMAX_SPLITS + sp] = mx;
    part_idx[r * ARGMAX_SPLITS + sp] = s_idx;
    __threadfence();
    s_last = atomicAdd(&tickets[r], 1) == ARGMAX_SPLITS - 1;
  }
  __syncthreads();
  if (!s_last || threadIdx.x >= 32) return;
  __threadfence();
  float m = __ldcg(part_max + r * ARGMAX_SPLITS + threadIdx.x);     // ARGMAX_SPLITS == 32: one per lane
  int idx = __ldcg(part_idx + r * ARGMAX_SPLITS + threadIdx.x);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
    if (m2 > m || (m2 == m && i2 < idx)) { m = m2; idx = i2; }
  }
  if (threadIdx.x == 0) {
    out[r] = idx == 0x7fffffff ? 0 : idx;
    tickets[r] = 0;
  }
}

// Words of scratch (4 bytes each) that si_argmax needs for up to `capacity` rows; the caller zeroes them
// once. The tickets stand first, so that they lie in the same place for every number of rows.
SI_EXPORT long long si_argmax_scratch_words(int capacity) { return (long long)capacity * (2 * ARGMAX_SPLITS + 1); }

SI_EXPORT int si_argmax(const float* logits, long long row_stride, int num_rows, int vocab, void* scratch, int capacity,
                        int* out, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (!scratch || num_rows > capacity || num_rows > 65535) return -2;
  int* tickets = (int*)scratch;
  float* part_max = (float*)scratch + capacity;
  int* part_idx = (int*)scratch + capacity + (size_t)capacity * ARGMAX_SPLITS;
  si_launch(argmax_split_kernel, dim3(ARGMAX_SPLITS, num_rows), dim3(ARGMAX_THREADS), 0, stream, logits, row_stride,
            vocab, part_max, part_idx, tickets, out);
  return si_last_error();
}

SI_EXPORT int si_sample(const float* logits, long long row_stride, int num_rows, int vocab,
                        const float* temperature, const int* top_k, const float* top_p,
                        const unsigned long long* seed, const unsigned long long* counter,
                        int* out, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  si_launch(sample_kernel, dim3(num_rows), dim3(SAMPLE_THREADS), 0, stream, logits, row_stride, vocab, temperature,
            top_k, top_p, seed, counter, out);
  return si_last_error();
}
