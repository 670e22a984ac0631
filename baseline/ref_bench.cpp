// Driver for the reference arm of bench.py: runs the UNMODIFIED reference project (compiled in place from its
// own sources, continuous KV layout, i.e. its CMake option USE_PAGED_ATTENTION off) through its own public
// classes on the GPU and prints one JSON object. Nothing of this repository's engine is linked or called.
//
//   ref_bench verify <model.bin> <max_seq> <prompt file>
//       greedy tokens of two requests through scheduler::Scheduler on the CUDA device ("SEQ <id> gen: ..."),
//       for comparison with the tokens its CPU device gave (tests/golden).
//   ref_bench bench <model.bin> <batch> <ctx> <steps> <warmup> <sched_rows> <ctx2>
//       value: model::Model::decode_step (its CUDA-graph decode path) on `batch` sequences whose contexts end
//              near `ctx`, timed on the device with CUDA events around `steps` steps after `warmup`;
//       e2e:   the same steps with host tokens in and sampled tokens out every step (decode_step, stream sync,
//              post_processing_batch: what its Scheduler runs for a decode step);
//       and `batch` prompts of 4/5 of `ctx2` tokens through scheduler::Scheduler itself (`sched_rows` = its
//       max_batch_size, the rows of a step), timed while all of them decode.
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
  if (argc < 9) return 2;
  const char* bin = argv[2];
  const int batch = atoi(argv[3]), ctx = atoi(argv[4]), steps = atoi(argv[5]), warm = atoi(argv[6]);
  const int rows = atoi(argv[7]), ctx2 = atoi(argv[8]);      // scheduler run: rows a step, context of the short workload
  auto m = load(bin);
  const int L = m->layer_num(), kvd = m->kv_dim(), V = m->vocab_size();
  if (ctx > m->seq_len() || batch < 1 || steps < 1 || rows < batch) {
    printf("{\"error\": \"bad sizes\"}\n");
    return 2;
  }
  // The reference forms a tensor's size as a product of 32-bit ints (src/source/tensor/tensor.cpp:85).
  if ((long long)L * batch * kvd * ctx >= (1ll << 31)) {
    printf("{\"error\": \"cache of %d x %d x %d x %d elements overflows the reference's 32-bit tensor size\"}\n", L, batch, kvd, ctx);
    return 5;
  }
  auto cu = base::CUDADeviceAllocatorFactory::get_instance();
  auto cpu = base::CPUDeviceAllocatorFactory::get_instance();
  double dev_ms = 0.0, e2e_s = 0.0;
  {
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
    // ---- value: device-timed decode steps through Model::decode_step -----------------------------------
    const int start = ctx - 2 * (steps + warm) - 2;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    unsigned rng = 12345u;
    int p = start;
    for (int i = 0; i < warm + steps; ++i, ++p) {
      if (i == warm) {
        m->sync_stream();
        cudaEventRecord(e0, 0);
      }
      for (int b = 0; b < batch; ++b) {
        rng = rng * 1664525u + 1013904223u;
        ids.ptr<int32_t>()[b] = (int)((rng >> 8) % (unsigned)V);
        pos.ptr<int32_t>()[b] = p;
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
    // ---- e2e: what its Scheduler does in a decode step (scheduler.cpp:557-610): host tokens and positions in,
    // decode_step, stream sync, post_processing_batch (argmax kernel, token ids back to the host), and the
    // sampled tokens are the next step's inputs. The Scheduler itself cannot hold this workload: it caps the
    // rows of a step, prompt rows included, at max_batch, which also sizes the cache.
    std::vector<int32_t> next(batch, 1);
    auto one = [&]() {
      for (int b = 0; b < batch; ++b) {
        ids.ptr<int32_t>()[b] = next[b];
        pos.ptr<int32_t>()[b] = p;
        slots.ptr<int32_t>()[b] = b;
      }
      ++p;
      auto st = m->decode_step(ids, pos, slots, kc, vc, logits);
      if (!st) return false;
      m->sync_stream();
      next = m->post_processing_batch(logits);
      return true;
    };
    for (int i = 0; i < 2; ++i)
      if (!one()) { printf("{\"error\": \"decode_step failed\"}\n"); return 6; }
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < steps; ++i)
      if (!one()) { printf("{\"error\": \"decode_step failed\"}\n"); return 6; }
    e2e_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (!cuda_ok("the end-to-end loop")) return 4;
  }
  cu->free_idle();

  // ---- the short workload through the Scheduler itself: `batch` prompts of ctx2 * 4 / 5 tokens. Its prompts go in
  // one after the other (rows of a step are capped at `rows`), so the first request has generated some hundred
  // tokens when the last one starts to decode: the requests get room to generate 3/5 of ctx2, and `steps` steps
  // are timed from the moment all of them decode (their contexts then lie between 4/5 and about ctx2).
  double sched_tps = 0.0, sched_ms = 0.0, sched_ctx = 0.0;
  long sched_steps = 0, prefill_steps = 0;
  const int cap2 = ctx2 * 7 / 5;
  if (ctx2 > 0 && (long long)L * rows * kvd * cap2 < (1ll << 31) && cap2 <= m->seq_len()) {
    const int plen = ctx2 * 4 / 5;
    scheduler::Scheduler s(m, rows, cap2, cap2 - plen, 0);
    unsigned rng = 777u;
    for (int j = 0; j < batch; ++j) {
      std::vector<int> prompt(plen);
      for (auto& t : prompt) {
        rng = rng * 1664525u + 1013904223u;
        t = (int)((rng >> 8) % (unsigned)V);
      }
      if (s.add_request(prompt) < 0) {
        printf("{\"error\": \"request rejected\"}\n");
        return 7;
      }
    }
    auto all_decoding = [&]() {
      if ((int)s.get_running().size() != batch) return false;
      for (auto& q : s.get_running())
        if (!q.is_prefill_complete || q.generated_tokens.empty()) return false;
      return true;
    };
    while (!all_decoding()) {
      s.step();
      if (++prefill_steps > 1000000 || (s.get_running().empty() && s.num_waiting() == 0)) {
        printf("{\"error\": \"the scheduler never reached %d decoding requests\"}\n", batch);
        return 8;
      }
    }
    for (int i = 0; i < 3; ++i) s.step();
    m->sync_stream();
    for (auto& q : s.get_running()) sched_ctx += q.total_tokens() / (double)batch;
    auto t0 = std::chrono::steady_clock::now();
    while ((int)s.get_running().size() == batch && sched_steps < steps) {
      s.step();
      ++sched_steps;
    }
    m->sync_stream();
    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    sched_tps = (double)batch * sched_steps / dt;
    sched_ms = dt * 1e3 / (sched_steps ? sched_steps : 1);
    if (!cuda_ok("the scheduler steps")) return 4;
  }
  printf("{\"device_ms\": %.4f, \"steps\": %d, \"batch\": %d, \"context\": %d, \"e2e_s\": %.6f, \"e2e_tokens\": %ld, "
         "\"h2d_bytes_per_step\": %d, \"d2h_bytes_per_step\": %d, \"sched_context\": %d, \"sched_rows\": %d, "
         "\"sched_prefill_steps\": %ld, \"sched_decode_steps\": %ld, \"sched_tokens_per_s\": %.1f, \"sched_ms_per_step\": %.4f, "
         "\"sched_mean_context\": %.1f}\n",
         dev_ms, steps, batch, ctx, e2e_s, (long)batch * steps, 3 * batch * 4, batch * 4, ctx2, rows, prefill_steps,
         sched_steps, sched_tps, sched_ms, sched_ctx + sched_steps / 2.0);
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
