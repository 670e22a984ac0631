// Driver for the reference arm of bench.py: runs the UNMODIFIED reference project (compiled in place from its
// own sources, continuous KV layout, i.e. its CMake option USE_PAGED_ATTENTION off) through its own public
// classes on the GPU and prints one JSON object. Nothing of this repository's engine is linked or called.
//
//   ref_bench verify <model.bin> <max_seq> <prompt file>
//       greedy tokens of two requests through scheduler::Scheduler on the CUDA device ("SEQ <id> gen: ..."),
//       for comparison with the tokens its CPU device gave (tests/golden).
//   ref_bench bench <model.bin> <batch> <ctx> <steps> <warmup> <sched_rows>
//       value: model::Model::decode_step (its CUDA-graph decode path) on `batch` sequences whose contexts end
//              at `ctx`, timed on the device with CUDA events around `steps` steps after `warmup`;
//       e2e:   the same workload through scheduler::Scheduler::step (host tokens in, sampled tokens out every
//              step), prompts prefilled by the scheduler itself, `sched_rows` = its max_batch_size (rows a step).
#include "model/llama3.h"
#include "scheduler/scheduler.h"
#include <base/alloc.h>
#include <cuda_runtime_api.h>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

static std::shared_ptr<model::LLamaModel> load(const char* bin) {
  auto m = std::make_shared<model::LLamaModel>(base::TokenizerType::kEncodeSpe, "tok", bin, false);
  auto st = m->init(base::DeviceType::kDeviceCUDA);
  if (!st) {
    printf("{\"error\": \"init failed: %s\"}\n", st.get_err_msg().c_str());
    exit(3);
  }
  return m;
}

static int cuda_ok(const char* where) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    printf("{\"error\": \"CUDA error after %s: %s\"}\n", where, cudaGetErrorString(e));
    return 0;
  }
  return 1;
}

static int verify(int argc, char** argv) {
  if (argc < 5) return 2;
  auto m = load(argv[2]);
  int max_seq = atoi(argv[3]);
  std::vector<int> prompt;
  FILE* f = fopen(argv[4], "r");
  int t;
  while (f && fscanf(f, "%d", &t) == 1) prompt.push_back(t);
  if (f) fclose(f);
  scheduler::Scheduler s(m, 4, max_seq, 8, max_seq);
  s.add_request(prompt);
  std::vector<int> p2(prompt.begin(), prompt.begin() + 3);
  s.add_request(p2);
  int guard = 0;
  while (!s.all_finished() && guard++ < 10000) s.step();
  if (!cuda_ok("the scheduler run")) return 4;
  for (auto& q : s.get_finished()) {
    printf("SEQ %d gen:", q.id);
    for (int g : q.generated_tokens) printf(" %d", g);
    printf("\n");
  }
  return 0;
}

static int bench(int argc, char** argv) {
  if (argc < 8) return 2;
  const char* bin = argv[2];
  const int batch = atoi(argv[3]), ctx = atoi(argv[4]), steps = atoi(argv[5]), warm = atoi(argv[6]);
  const int rows = atoi(argv[7]);
  auto m = load(bin);
  const int L = m->layer_num(), kvd = m->kv_dim(), V = m->vocab_size();
  if (ctx > m->seq_len() || batch < 1 || steps < 1 || rows < batch) {
    printf("{\"error\": \"bad sizes\"}\n");
    return 2;
  }
  auto cu = base::CUDADeviceAllocatorFactory::get_instance();
  auto cpu = base::CPUDeviceAllocatorFactory::get_instance();
  double dev_ms = 0.0;
  {
    // ---- device-timed decode steps through Model::decode_step ------------------------------------------
    tensor::Tensor kc(base::DataType::kDataTypeFp32, L, batch, kvd, ctx, true, cu);
    tensor::Tensor vc(base::DataType::kDataTypeFp32, L, batch, kvd, ctx, true, cu);
    tensor::Tensor logits(base::DataType::kDataTypeFp32, batch, V, true, cu);
    if (kc.is_empty() || vc.is_empty() || logits.is_empty()) {
      printf("{\"error\": \"cache allocation failed\"}\n");
      return 5;
    }
    const size_t cache_bytes = (size_t)L * batch * kvd * ctx * sizeof(float);
    cudaMemset(kc.ptr<float>(), 0, cache_bytes);
    cudaMemset(vc.ptr<float>(), 0, cache_bytes);
    tensor::Tensor ids(base::DataType::kDataTypeInt32, batch, true, cpu), pos(base::DataType::kDataTypeInt32, batch, true, cpu),
        slots(base::DataType::kDataTypeInt32, batch, true, cpu);
    const int start = ctx - (steps + warm) - 1;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    unsigned rng = 12345u;
    for (int i = 0; i < warm + steps; ++i) {
      if (i == warm) {
        m->sync_stream();
        cudaEventRecord(e0, 0);
      }
      for (int b = 0; b < batch; ++b) {
        rng = rng * 1664525u + 1013904223u;
        ids.ptr<int32_t>()[b] = (int)((rng >> 8) % (unsigned)V);
        pos.ptr<int32_t>()[b] = start + i;
        slots.ptr<int32_t>()[b] = b;
      }
      auto st = m->decode_step(ids, pos, slots, kc, vc, logits);
      if (!st) {
        printf("{\"error\": \"decode_step failed: %s\"}\n", st.get_err_msg().c_str());
        return 6;
      }
    }
    cudaEventRecord(e1, 0);        // the legacy default stream waits for the model's (blocking) stream
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    dev_ms = ms;
    if (!cuda_ok("the decode_step loop")) return 4;
  }
  cu->free_idle();

  // ---- end to end through the Scheduler ------------------------------------------------------------------
  // Prompts are staggered so that, when the last one has been prefilled, every request stands at about the same
  // context: request j's prompt takes about ceil(P_j / (rows - j)) steps while the j requests before it decode.
  const int T0 = ctx - (steps + warm) - 8;
  std::vector<int> P(batch);
  {
    long after = 0;
    for (int j = batch - 1; j >= 0; --j) {
      P[j] = (int)std::max<long>(16, T0 - after);
      after += (P[j] + (rows - j) - 1) / (rows - j);
    }
  }
  scheduler::Scheduler s(m, rows, ctx, ctx, 0);
  unsigned rng = 777u;
  for (int j = 0; j < batch; ++j) {
    std::vector<int> prompt(P[j]);
    for (auto& t : prompt) {
      rng = rng * 1664525u + 1013904223u;
      t = (int)((rng >> 8) % (unsigned)V);
    }
    if (s.add_request(prompt) < 0) {
      printf("{\"error\": \"request rejected\"}\n");
      return 7;
    }
  }
  long prefill_steps = 0;
  auto all_decoding = [&]() {
    if ((int)s.get_running().size() != batch) return false;
    for (auto& q : s.get_running())
      if (!q.is_prefill_complete || q.generated_tokens.empty()) return false;
    return true;
  };
  auto t_pre = std::chrono::steady_clock::now();
  while (!all_decoding()) {
    s.step();
    if (++prefill_steps > 2000000 || (s.get_running().empty() && s.num_waiting() == 0)) {
      printf("{\"error\": \"the scheduler never reached %d decoding requests\"}\n", batch);
      return 8;
    }
  }
  double prefill_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_pre).count();
  for (int i = 0; i < warm; ++i) s.step();
  auto tokens_now = [&]() {
    long n = 0;
    for (auto& q : s.get_running()) n += q.num_generated_tokens;
    for (auto& q : s.get_finished()) n += q.num_generated_tokens;
    return n;
  };
  double ctx_sum = 0;
  for (auto& q : s.get_running()) ctx_sum += q.total_tokens();
  const double ctx_start = ctx_sum / batch;
  m->sync_stream();
  const long n0 = tokens_now();
  auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < steps; ++i) s.step();
  m->sync_stream();
  const double e2e_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  const long made = tokens_now() - n0;
  const int still = (int)s.get_running().size();
  if (!cuda_ok("the scheduler steps")) return 4;
  printf("{\"device_ms\": %.4f, \"steps\": %d, \"batch\": %d, \"e2e_s\": %.6f, \"e2e_tokens\": %ld, \"running_at_end\": %d, "
         "\"e2e_context_start\": %.1f, \"prefill_steps\": %ld, \"prefill_s\": %.2f, \"sched_rows\": %d, "
         "\"h2d_bytes_per_step\": %d, \"d2h_bytes_per_step\": %d}\n",
         dev_ms, steps, batch, e2e_s, made, still, ctx_start, prefill_steps, prefill_s, rows, 3 * batch * 4, batch * 4);
  fflush(stdout);
  _exit(0);      // skip the destructors of the reference's globals
}

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  std::string mode = argv[1];
  if (mode == "verify") return verify(argc, argv);
  if (mode == "bench") return bench(argc, argv);
  return 2;
}
