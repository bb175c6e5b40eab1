// Decode steps whose per-step inputs and result live in host memory (no counterpart in the
// reference, whose bindings take device tensors, paged_attention_loop/paged_attention_loop.cpp:21-38).
//   pa_decode_step_host        one upload, the launch, one download, in order on one stream
//   pa_decode_step_host_batch  the same step cut into sub-batches of consecutive sequences whose
//                              uploads, kernels and downloads overlap on three streams
#include <cmath>
#include <mutex>

#include "launch_common.cuh"

namespace pa {
namespace {

int launch_entry(int32_t entry, const pa_params *p, void *stream) {
  switch (entry) {
  case PA_ENTRY_LOOP: return launch_kernels_loop(p, stream, nullptr);
  case PA_ENTRY_REDUCE: return launch_kernels_reduce(p, stream, nullptr);
  case PA_ENTRY_FP8_LOOP: return launch_kernels_fp8_loop(p, stream, nullptr);
  default: return launch_kernels_fp8_reduce(p, stream, nullptr);
  }
}

constexpr uint32_t kMaxSubBatches = 8;

// Copy streams and events of the pipelined step, created on first use, one set per device.
struct StepResources {
  bool ready = false;
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t start = nullptr, out_done = nullptr;
  cudaEvent_t in_done[kMaxSubBatches] = {}, kernels_done[kMaxSubBatches] = {};
};

int step_resources(StepResources **out) {
  constexpr int kMaxDevices = 64;
  static StepResources table[kMaxDevices];
  static std::mutex mu;
  int device = 0;
  PA_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return fail(PA_ERR_CUDA, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(mu);
  StepResources &r = table[device];
  if (!r.ready) {
    PA_CUDA_TRY(cudaStreamCreateWithFlags(&r.copy_in, cudaStreamNonBlocking));
    PA_CUDA_TRY(cudaStreamCreateWithFlags(&r.copy_out, cudaStreamNonBlocking));
    PA_CUDA_TRY(cudaEventCreateWithFlags(&r.start, cudaEventDisableTiming));
    PA_CUDA_TRY(cudaEventCreateWithFlags(&r.out_done, cudaEventDisableTiming));
    for (uint32_t k = 0; k < kMaxSubBatches; ++k) {
      PA_CUDA_TRY(cudaEventCreateWithFlags(&r.in_done[k], cudaEventDisableTiming));
      PA_CUDA_TRY(cudaEventCreateWithFlags(&r.kernels_done[k], cudaEventDisableTiming));
    }
    r.ready = true;
  }
  *out = &r;
  return PA_OK;
}

template <typename T>
T *advance(T *base, size_t bytes) {
  return base == nullptr ? nullptr
                         : reinterpret_cast<T *>(reinterpret_cast<uintptr_t>(base) + bytes);
}

size_t table_entries_of(const pa_params *p, const pa_host_batch *io) {
  const uint32_t S = p->num_seqs;
  return io->host_block_table_offsets != nullptr
             ? static_cast<size_t>(io->host_block_table_offsets[S] - io->host_block_table_offsets[0])
             : static_cast<size_t>(S) * p->max_blocks_per_seq;
}

// Number of sub-batches of a pipelined step.  A further sub-batch costs about 40 us (the ramp
// and tail of one more launch pair, more copies and events); cutting into n hides (1 - 1/n) of
// the transfer time, about 16 us of latencies plus the bytes at the 25 GB/s per direction
// measured for pinned memory on B200 hosts.  The sum is smallest near
// n = sqrt(transfer time / 40 us) (measured: 4 for 17 MB per step, 3 for 2 MB, 1 below 1 MB).
uint32_t choose_sub_batches(const pa_params *p, const pa_host_batch *io) {
  const uint32_t S = p->num_seqs;
  uint32_t n = io->sub_batches;
  if (n == 0) {
    const double row_bytes = 2.0 * p->num_heads * p->head_size;
    const double bytes = 2.0 * row_bytes * S + 4.0 * (static_cast<double>(table_entries_of(p, io)) + 2.0 * S);
    const double transfer_us = 16.0 + bytes / 25.0e3;
    n = static_cast<uint32_t>(std::sqrt(transfer_us / 40.0) + 0.5);
    if (n == 2) n = 3; // from three pieces on the two end pieces are small (see the boundaries below)
  }
  return std::max(1u, std::min(std::min(n, kMaxSubBatches), std::max(S, 1u)));
}

// The step without sub-batches: uploads, launch and download in order on the caller's stream,
// no second stream and no events.  When the caller's host inputs are one staging block mirrored
// on the device (pa_host_batch.host_staging) the upload is a single copy.
int single_batch_step(int32_t entry, const pa_params *p, const pa_host_batch *io, bool packed, size_t row_bytes,
                      size_t table_entries, void *stream, int32_t synchronize) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint32_t S = p->num_seqs;
  if (io->host_staging != nullptr && io->dev_staging != nullptr && io->staging_bytes != 0) {
    PA_CUDA_TRY(cudaMemcpyAsync(io->dev_staging, io->host_staging, io->staging_bytes, cudaMemcpyHostToDevice, st));
  } else {
    PA_CUDA_TRY(cudaMemcpyAsync(const_cast<void *>(p->query), io->host_query, S * row_bytes, cudaMemcpyHostToDevice, st));
    PA_CUDA_TRY(cudaMemcpyAsync(const_cast<uint32_t *>(p->context_lens), io->host_context_lens, S * sizeof(uint32_t),
                                cudaMemcpyHostToDevice, st));
    if (packed)
      PA_CUDA_TRY(cudaMemcpyAsync(const_cast<uint32_t *>(p->block_table_offsets), io->host_block_table_offsets,
                                  (S + 1) * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
    if (table_entries != 0) {
      const size_t first = packed ? io->host_block_table_offsets[0] : 0;
      PA_CUDA_TRY(cudaMemcpyAsync(const_cast<uint32_t *>(p->block_tables) + first, io->host_block_tables + first,
                                  table_entries * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
    }
  }
  const bool direct = (io->flags & PA_STEP_LAST_OUT_DIRECT) != 0u;
  pa_params whole = *p;
  if (direct) whole.out = io->host_out;
  if (int rc = launch_entry(entry, &whole, stream)) return rc;
  if (!direct) PA_CUDA_TRY(cudaMemcpyAsync(io->host_out, p->out, S * row_bytes, cudaMemcpyDeviceToHost, st));
  if (synchronize != 0) PA_CUDA_TRY(cudaStreamSynchronize(st));
  return PA_OK;
}

} // namespace
} // namespace pa

extern "C" {

PA_API int pa_split_by_kv_length(const uint32_t *context_lens, uint32_t num_seqs, uint32_t parts, uint32_t *bounds) {
  if (parts == 0 || bounds == nullptr || (num_seqs != 0 && context_lens == nullptr))
    return pa::fail(PA_ERR_BAD_ARG, "split: parts must be positive and the arrays non-null");
  uint64_t total = 0;
  for (uint32_t i = 0; i < num_seqs; ++i) total += context_lens[i];
  // part r ends behind the sequence whose cumulative length reaches (r + 1) / parts of the total
  uint64_t cum = 0;
  uint32_t r = 0;
  bounds[0] = 0;
  for (uint32_t i = 0; i < num_seqs; ++i) {
    cum += context_lens[i];
    while (r + 1 < parts && total > 0 && cum * parts >= static_cast<uint64_t>(r + 1) * total) bounds[++r] = i + 1;
  }
  while (r < parts) bounds[++r] = num_seqs;
  return PA_OK;
}

PA_API int pa_decode_step_host(int32_t entry, const pa_params *p, const pa_host_step *io, void *stream,
                               int32_t synchronize) {
  if (p == nullptr || io == nullptr) return pa::fail(PA_ERR_BAD_ARG, "params or host step is null");
  if (entry < PA_ENTRY_LOOP || entry > PA_ENTRY_FP8_REDUCE) return pa::fail(PA_ERR_BAD_ARG, "unknown entry %d", entry);
  if ((io->in_bytes != 0 && (io->host_in == nullptr || io->dev_in == nullptr)) ||
      (io->out_bytes != 0 && io->host_out == nullptr))
    return pa::fail(PA_ERR_BAD_ARG, "host step: a buffer with a non-zero size is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (io->in_bytes != 0)
    PA_CUDA_TRY(cudaMemcpyAsync(io->dev_in, io->host_in, io->in_bytes, cudaMemcpyHostToDevice, st));
  if (int rc = pa::launch_entry(entry, p, stream)) return rc;
  if (io->out_bytes != 0)
    PA_CUDA_TRY(cudaMemcpyAsync(io->host_out, p->out, io->out_bytes, cudaMemcpyDeviceToHost, st));
  if (synchronize != 0) PA_CUDA_TRY(cudaStreamSynchronize(st));
  return PA_OK;
}

PA_API int pa_host_batch_plan(const pa_params *p, const pa_host_batch *io, uint32_t *sub_batches,
                              uint64_t *h2d_bytes, uint64_t *d2h_bytes) {
  using namespace pa;
  if (p == nullptr || io == nullptr || io->host_context_lens == nullptr)
    return fail(PA_ERR_BAD_ARG, "params, host batch or its context lengths are null");
  const uint32_t S = p->num_seqs;
  const uint32_t n = choose_sub_batches(p, io);
  const uint64_t row_bytes = static_cast<uint64_t>(p->num_heads) * p->head_size * 2;
  uint64_t up = S * row_bytes + 4ull * S + 4ull * table_entries_of(p, io) +
                (io->host_block_table_offsets != nullptr ? 4ull * (S + 1) : 0ull);
  if (n == 1 && io->host_staging != nullptr && io->dev_staging != nullptr && io->staging_bytes != 0)
    up = io->staging_bytes;
  if (sub_batches) *sub_batches = n;
  if (h2d_bytes) *h2d_bytes = up;
  if (d2h_bytes) *d2h_bytes = S * row_bytes; // by the copy engine or, for a direct last sub-batch, by the kernels
  return PA_OK;
}

PA_API int pa_decode_step_host_batch(int32_t entry, const pa_params *p, const pa_host_batch *io, void *stream,
                                     int32_t synchronize) {
  using namespace pa;
  if (p == nullptr || io == nullptr) return fail(PA_ERR_BAD_ARG, "params or host batch is null");
  if (entry < PA_ENTRY_LOOP || entry > PA_ENTRY_FP8_REDUCE) return fail(PA_ERR_BAD_ARG, "unknown entry %d", entry);
  if (p->seq_indices != nullptr)
    return fail(PA_ERR_BAD_ARG, "host batch: sub-batches are ranges of consecutive sequences, seq_indices must be NULL");
  const uint32_t S = p->num_seqs;
  if (S == 0) return PA_OK;
  if (!io->host_query || !io->host_block_tables || !io->host_context_lens || !io->host_out || !p->query ||
      !p->block_tables || !p->context_lens || !p->out)
    return fail(PA_ERR_BAD_ARG, "host batch: a required host or device buffer is null");
  const bool packed = io->host_block_table_offsets != nullptr;
  if (packed != (p->block_table_offsets != nullptr))
    return fail(PA_ERR_BAD_ARG, "host batch: host and device block-table offsets must both be set or both be NULL");
  if (io->sub_batches > kMaxSubBatches) return fail(PA_ERR_BAD_ARG, "host batch: at most %u sub-batches", kMaxSubBatches);
  const bool reduce = entry == PA_ENTRY_REDUCE || entry == PA_ENTRY_FP8_REDUCE;
  const size_t row_bytes = static_cast<size_t>(p->num_heads) * p->head_size * 2; // one sequence of query / out
  const size_t table_entries = table_entries_of(p, io);
  const uint32_t n = choose_sub_batches(p, io);
  if (n == 1) return single_batch_step(entry, p, io, packed, row_bytes, table_entries, stream, synchronize);
  // ---- boundaries by KV tokens (the kernels' time follows the tokens).  The upload of the first
  // sub-batch and the download of the last are the only transfers nothing hides, so the two end
  // pieces are a third of the size of the inner ones (weights 1, 3, ..., 3, 1).
  uint32_t bound[kMaxSubBatches + 1];
  {
    const uint32_t inner = (n >= 3) ? 3u : 1u;
    const uint64_t weight_sum = 2ull + static_cast<uint64_t>(inner) * (n - 2u);
    uint64_t total = 0;
    for (uint32_t i = 0; i < S; ++i) total += io->host_context_lens[i];
    // piece r ends behind the sequence whose cumulative length reaches its cumulative weight
    uint64_t cum = 0, weight_done = 1; // cumulative weight up to and including piece r
    uint32_t rr = 0;
    bound[0] = 0;
    for (uint32_t i = 0; i < S; ++i) {
      cum += io->host_context_lens[i];
      while (rr + 1 < n && total > 0 && cum * weight_sum >= weight_done * total) {
        bound[++rr] = i + 1;
        weight_done += (rr + 1 < n) ? inner : 1u;
      }
    }
    while (rr < n) bound[++rr] = S;
  }
  StepResources *r = nullptr;
  if (int rc = step_resources(&r)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the previous work of `stream` may still read the device mirrors: uploads start after it
  PA_CUDA_TRY(cudaEventRecord(r->start, st));
  PA_CUDA_TRY(cudaStreamWaitEvent(r->copy_in, r->start, 0));
  const bool direct_last = (io->flags & PA_STEP_LAST_OUT_DIRECT) != 0u;
  bool any_copy_out = false;
  uint32_t next_offset = 0; // packed tables: first row offset that has not gone up yet
  for (uint32_t k = 0; k < n; ++k) {
    const uint32_t lo = bound[k], hi = bound[k + 1];
    if (hi <= lo) continue;
    const uint32_t cnt = hi - lo;
    // ---- upload of the sub-batch's inputs
    PA_CUDA_TRY(cudaMemcpyAsync(advance(const_cast<void *>(p->query), lo * row_bytes),
                                advance(io->host_query, lo * row_bytes), cnt * row_bytes, cudaMemcpyHostToDevice,
                                r->copy_in));
    PA_CUDA_TRY(cudaMemcpyAsync(const_cast<uint32_t *>(p->context_lens) + lo, io->host_context_lens + lo,
                                cnt * sizeof(uint32_t), cudaMemcpyHostToDevice, r->copy_in));
    if (packed) {
      const uint32_t *off = io->host_block_table_offsets;
      // offsets [lo, hi]; offsets[lo] has gone up with the previous sub-batch unless this is the first
      PA_CUDA_TRY(cudaMemcpyAsync(const_cast<uint32_t *>(p->block_table_offsets) + next_offset, off + next_offset,
                                  (hi + 1 - next_offset) * sizeof(uint32_t), cudaMemcpyHostToDevice, r->copy_in));
      next_offset = hi + 1;
      if (off[hi] > off[lo])
        PA_CUDA_TRY(cudaMemcpyAsync(const_cast<uint32_t *>(p->block_tables) + off[lo], io->host_block_tables + off[lo],
                                    static_cast<size_t>(off[hi] - off[lo]) * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                    r->copy_in));
    } else {
      const size_t mb = p->max_blocks_per_seq;
      PA_CUDA_TRY(cudaMemcpyAsync(const_cast<uint32_t *>(p->block_tables) + lo * mb, io->host_block_tables + lo * mb,
                                  cnt * mb * sizeof(uint32_t), cudaMemcpyHostToDevice, r->copy_in));
    }
    PA_CUDA_TRY(cudaEventRecord(r->in_done[k], r->copy_in));
    PA_CUDA_TRY(cudaStreamWaitEvent(st, r->in_done[k], 0));
    // ---- the sub-batch is the same call with every per-sequence pointer moved to its first row
    pa_params sub = *p;
    sub.num_seqs = cnt;
    sub.query = advance(p->query, lo * row_bytes);
    sub.out = advance(p->out, lo * row_bytes);
    sub.context_lens = p->context_lens + lo;
    if (packed) sub.block_table_offsets = p->block_table_offsets + lo;
    else sub.block_tables = p->block_tables + static_cast<size_t>(lo) * p->max_blocks_per_seq;
    if (reduce) {
      const size_t stat_rows = static_cast<size_t>(lo) * p->num_heads * p->max_num_partitions;
      sub.max_logits = advance(p->max_logits, stat_rows * sizeof(float));
      sub.exp_sums = advance(p->exp_sums, stat_rows * sizeof(float));
      sub.tmp_out = advance(p->tmp_out, stat_rows * p->head_size * 2);
    }
    const bool direct = direct_last && k + 1 == n;
    if (direct) sub.out = advance(io->host_out, lo * row_bytes); // the kernels write the host buffer themselves
    if (int rc = launch_entry(entry, &sub, stream)) return rc;
    if (!direct) {
      PA_CUDA_TRY(cudaEventRecord(r->kernels_done[k], st));
      PA_CUDA_TRY(cudaStreamWaitEvent(r->copy_out, r->kernels_done[k], 0));
      PA_CUDA_TRY(cudaMemcpyAsync(advance(io->host_out, lo * row_bytes), advance(p->out, lo * row_bytes),
                                  cnt * row_bytes, cudaMemcpyDeviceToHost, r->copy_out));
      any_copy_out = true;
    }
  }
  if (any_copy_out) {
    // join: whatever follows on `stream` (and the wait below) sees every download finished
    PA_CUDA_TRY(cudaEventRecord(r->out_done, r->copy_out));
    PA_CUDA_TRY(cudaStreamWaitEvent(st, r->out_done, 0));
  }
  if (synchronize != 0) PA_CUDA_TRY(cudaStreamSynchronize(st));
  return PA_OK;
}

} // extern "C"
