// Embedding gather: out[t, :] = table[tokens[t], :], widened to fp32 (the residual
// stream is fp32 in both precisions). The reference's kernel
// (src/source/op/kernels/cuda/emb_kernel.cu:3-21) silently skips token ids outside
// the vocabulary; here such a row is zeroed and the status word is set.
#include "common.cuh"

template <typename TW>
__global__ void embedding_gather_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                        float* __restrict__ out, int hidden, int vocab,
                                        int* status) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  float* o = out + (size_t)t * hidden;
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) set_status(status, SI_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* w = table + (size_t)tok * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32<TW>(w[i]);
}

SI_EXPORT int si_embedding_gather(const int* tokens, const void* table, int table_dtype, float* out,
                                  int num_tokens, int hidden, int vocab, int* status,
                                  cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == SI_BF16)
    si_launch(embedding_gather_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream,
              tokens, (const __nv_bfloat16*)table, out, hidden, vocab, status);
  else
    si_launch(embedding_gather_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream,
              tokens, (const float*)table, out, hidden, vocab, status);
  return si_last_error();
}
