// Multi-GPU driver of the decode path (no counterpart in the reference, which is single-device:
// every call builds its own queue, paged_attention_loop/launch_kernels_loop.h:32-34).
//
// The path shards with no exchange step: every (sequence, KV head) is independent.  A caller that
// holds one batch gives every GPU a shard (sequences dealt by KV length, or a slice of the KV
// heads), each with its own KV pool, tables, queries and outputs on that GPU.  The driver runs
// the shards from ONE process: one host thread and one stream per shard, a common start barrier,
// device-side timing per shard, and reports the slowest shard, max_g(t_g).  No collective, no
// peer access on the data path: every GPU reads its own HBM only.  The optional gather of the
// (small) outputs onto one GPU runs after the timed region.
#include <chrono>
#include <condition_variable>
#include <mutex>
#include <thread>
#include <vector>

#include "launch_common.cuh"

namespace pa {
namespace {

// all threads wait until `count` of them have arrived; reusable
class HostBarrier {
public:
  explicit HostBarrier(uint32_t count) : count_(count) {}
  void arrive_and_wait() {
    std::unique_lock<std::mutex> lock(mu_);
    const uint64_t round = round_;
    if (++arrived_ == count_) {
      arrived_ = 0;
      ++round_;
      cv_.notify_all();
    } else {
      cv_.wait(lock, [&] { return round_ != round; });
    }
  }

private:
  std::mutex mu_;
  std::condition_variable cv_;
  uint32_t count_, arrived_ = 0;
  uint64_t round_ = 0;
};

struct ShardOutcome {
  int rc = PA_OK;
  float us_per_call = 0.f;
  char message[320] = "";
};

int default_launch(int32_t entry, const pa_params *p, void *stream, void *) {
  switch (entry) {
  case PA_ENTRY_LOOP: return launch_kernels_loop(p, stream, nullptr);
  case PA_ENTRY_REDUCE: return launch_kernels_reduce(p, stream, nullptr);
  case PA_ENTRY_FP8_LOOP: return launch_kernels_fp8_loop(p, stream, nullptr);
  case PA_ENTRY_FP8_REDUCE: return launch_kernels_fp8_reduce(p, stream, nullptr);
  default: return fail(PA_ERR_BAD_ARG, "unknown entry %d", entry);
  }
}

void note_failure(ShardOutcome &out, int rc, const char *what) {
  if (out.rc != PA_OK) return; // keep the first failure
  out.rc = rc;
  std::snprintf(out.message, sizeof(out.message), "%s", what);
}

#define PA_SHARD_CUDA(expr)                                                          \
  do {                                                                               \
    cudaError_t e__ = (expr);                                                        \
    if (e__ != cudaSuccess && out.rc == PA_OK) {                                     \
      char buf__[256];                                                               \
      std::snprintf(buf__, sizeof(buf__), "%s failed: %s", #expr, cudaGetErrorString(e__)); \
      note_failure(out, PA_ERR_CUDA, buf__);                                         \
    }                                                                                \
  } while (0)

void run_shard(const pa_device_shard &shard, const pa_multi_gpu_options &opt, HostBarrier &barrier,
               ShardOutcome &out) {
  const bool host_only = (opt.flags & PA_MULTI_GPU_HOST_ONLY) != 0u;
  pa_shard_launch_fn launch = opt.launch != nullptr ? opt.launch : default_launch;
  cudaStream_t stream = nullptr;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  if (!host_only) {
    PA_SHARD_CUDA(cudaSetDevice(shard.device));
    if (out.rc == PA_OK) PA_SHARD_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    if (out.rc == PA_OK) PA_SHARD_CUDA(cudaEventCreate(&t0));
    if (out.rc == PA_OK) PA_SHARD_CUDA(cudaEventCreate(&t1));
  }
  auto call = [&]() {
    if (out.rc != PA_OK) return;
    const int rc = launch(shard.entry, &shard.params, stream, opt.user);
    if (rc != PA_OK) note_failure(out, rc, opt.launch != nullptr ? "the launcher reported a failure" : last_error());
  };
  for (uint32_t i = 0; i < opt.warmup; ++i) call();
  if (!host_only && out.rc == PA_OK) PA_SHARD_CUDA(cudaStreamSynchronize(stream));
  // every shard arrives, also one that has failed: the others must not wait for it for ever
  barrier.arrive_and_wait();
  const auto h0 = std::chrono::steady_clock::now();
  if (!host_only && out.rc == PA_OK) PA_SHARD_CUDA(cudaEventRecord(t0, stream));
  for (uint32_t i = 0; i < opt.calls; ++i) call();
  if (!host_only && out.rc == PA_OK) PA_SHARD_CUDA(cudaEventRecord(t1, stream));
  if (!host_only && out.rc == PA_OK) PA_SHARD_CUDA(cudaEventSynchronize(t1));
  if (out.rc == PA_OK) {
    if (host_only) {
      const std::chrono::duration<double, std::micro> dt = std::chrono::steady_clock::now() - h0;
      out.us_per_call = static_cast<float>(dt.count() / opt.calls);
    } else {
      float ms = 0.f;
      PA_SHARD_CUDA(cudaEventElapsedTime(&ms, t0, t1));
      out.us_per_call = ms * 1000.f / static_cast<float>(opt.calls);
    }
  }
  barrier.arrive_and_wait(); // common end: nobody tears down while another shard still runs
  if (t0) cudaEventDestroy(t0);
  if (t1) cudaEventDestroy(t1);
  if (stream) cudaStreamDestroy(stream);
}

} // namespace
} // namespace pa

extern "C" {

PA_API int pa_multi_gpu_run(const pa_device_shard *shards, uint32_t num_shards, const pa_multi_gpu_options *options,
                            float *us_per_call_max, float *us_per_call_each) {
  using namespace pa;
  if (shards == nullptr || num_shards == 0 || options == nullptr || options->calls == 0)
    return fail(PA_ERR_BAD_ARG, "multi-GPU run: shards, options and a positive number of calls are required");
  if (num_shards > 64) return fail(PA_ERR_BAD_ARG, "multi-GPU run: at most 64 shards");
  int previous_device = -1;
  const bool host_only = (options->flags & PA_MULTI_GPU_HOST_ONLY) != 0u;
  if (!host_only) cudaGetDevice(&previous_device);
  HostBarrier barrier(num_shards);
  std::vector<ShardOutcome> outcome(num_shards);
  std::vector<std::thread> workers;
  workers.reserve(num_shards);
  for (uint32_t i = 0; i < num_shards; ++i)
    workers.emplace_back([&, i] { run_shard(shards[i], *options, barrier, outcome[i]); });
  for (auto &w : workers) w.join();
  if (!host_only && previous_device >= 0) cudaSetDevice(previous_device);
  float worst = 0.f;
  for (uint32_t i = 0; i < num_shards; ++i) {
    if (us_per_call_each != nullptr) us_per_call_each[i] = outcome[i].us_per_call;
    worst = std::max(worst, outcome[i].us_per_call);
  }
  if (us_per_call_max != nullptr) *us_per_call_max = worst;
  // aggregate: the first failing shard decides the code, the message names every failing shard
  int rc = PA_OK;
  char text[480] = "";
  size_t used = 0;
  for (uint32_t i = 0; i < num_shards; ++i) {
    if (outcome[i].rc == PA_OK) continue;
    if (rc == PA_OK) rc = outcome[i].rc;
    const int n = std::snprintf(text + used, sizeof(text) - used, "%sshard %u (device %d): %s", used ? "; " : "", i,
                                shards[i].device, outcome[i].message);
    if (n > 0) used = std::min(sizeof(text) - 1, used + static_cast<size_t>(n));
  }
  if (rc != PA_OK) return fail(rc, "%s", text);
  return PA_OK;
}

PA_API int pa_multi_gpu_gather_out(const pa_device_shard *shards, uint32_t num_shards, int32_t mode,
                                   void *dst, int32_t dst_device, uint32_t dst_num_heads) {
  using namespace pa;
  if (shards == nullptr || num_shards == 0 || dst == nullptr)
    return fail(PA_ERR_BAD_ARG, "gather: shards and a destination are required");
  if (mode != PA_GATHER_BY_SEQUENCE && mode != PA_GATHER_BY_KV_HEAD) return fail(PA_ERR_BAD_ARG, "gather: unknown mode %d", mode);
  int previous_device = -1;
  PA_CUDA_TRY(cudaGetDevice(&previous_device));
  PA_CUDA_TRY(cudaSetDevice(dst_device));
  size_t row_offset = 0;  // by sequence: rows of the shards follow one another
  size_t head_offset = 0; // by KV head: every shard holds all sequences and a slice of the heads
  int rc = PA_OK;
  for (uint32_t i = 0; i < num_shards && rc == PA_OK; ++i) {
    const pa_params &p = shards[i].params;
    const size_t row_bytes = static_cast<size_t>(p.num_heads) * p.head_size * 2;
    cudaError_t err;
    if (mode == PA_GATHER_BY_SEQUENCE) {
      err = cudaMemcpyPeerAsync(static_cast<char *>(dst) + row_offset, dst_device, p.out, shards[i].device,
                                row_bytes * p.num_seqs, nullptr);
      row_offset += row_bytes * p.num_seqs;
    } else {
      const size_t dst_pitch = static_cast<size_t>(dst_num_heads) * p.head_size * 2;
      err = cudaMemcpy2DAsync(static_cast<char *>(dst) + head_offset, dst_pitch, p.out, row_bytes, row_bytes,
                              p.num_seqs, cudaMemcpyDefault, nullptr);
      head_offset += row_bytes;
    }
    if (err != cudaSuccess) rc = fail(PA_ERR_CUDA, "gather of shard %u failed: %s", i, cudaGetErrorString(err));
  }
  if (rc == PA_OK) {
    const cudaError_t err = cudaStreamSynchronize(nullptr);
    if (err != cudaSuccess) rc = fail(PA_ERR_CUDA, "gather failed: %s", cudaGetErrorString(err));
  }
  cudaSetDevice(previous_device);
  return rc;
}

PA_API int pa_split_lpt(const uint32_t *context_lens, uint32_t num_seqs, uint32_t parts, uint32_t *part_of) {
  if (parts == 0 || part_of == nullptr || (num_seqs != 0 && context_lens == nullptr))
    return pa::fail(PA_ERR_BAD_ARG, "split: parts must be positive and the arrays non-null");
  // longest sequence first, each to the part that is lightest so far; ties go to the lower
  // sequence id and the lower part, so every caller computes the same answer
  std::vector<uint32_t> order(num_seqs);
  for (uint32_t i = 0; i < num_seqs; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return context_lens[a] > context_lens[b]; });
  std::vector<uint64_t> load(parts, 0);
  for (uint32_t i : order) {
    uint32_t best = 0;
    for (uint32_t r = 1; r < parts; ++r)
      if (load[r] < load[best]) best = r;
    load[best] += context_lens[i];
    part_of[i] = best;
  }
  return PA_OK;
}

} // extern "C"
