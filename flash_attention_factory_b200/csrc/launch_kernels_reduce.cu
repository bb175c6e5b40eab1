// launch_kernels_reduce: fp16 KV cache, split-context decode attention
// (per-partition attention kernel + merge kernel).  Host counterpart of the
// reference's dispatch_paged_attention / launch_paged_attn_v2
// (paged_attention_reduce/launch_kernels_reduce.h:18-78,80-197).
#include <mutex>

#include "launch_common.cuh"

namespace pa {
int read_status_reduce(int *v) { return read_and_clear_device_status(v); }
} // namespace pa

PA_TIMELINE_ACCESSOR(pa_debug_timeline_reduce)
PA_BOUNDS_ACCESSOR(pa_debug_bounds_reduce)

extern "C" PA_API int launch_kernels_reduce(const pa_params *p, void *stream, float *us_out) {
  using namespace pa;
  if (int rc = validate_params(p, /*fp8_entry=*/false, /*needs_scratch=*/true)) return rc;
  if (us_out) us_out[0] = us_out[1] = 0.f;
  if (p->num_seqs == 0) return PA_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return run_timed(
      s, us_out, [&] { return dispatch_head_size<KV_F16, MODE_SPLIT>(p, s); },
      [&] { return dispatch_merge(p, s); }, true);
}

// ----------------------------------------------------------------------------------------
// Split-context attention for callers that have no way to allocate device memory.
//
// Some hosts of this library cannot provide the three scratch tensors the split variant
// needs: a serving loop that has handed all of its device memory to a pool it does not own,
// a plugin running inside another runtime that forbids cudaMalloc after start-up, or code
// that must not trigger the implicit device synchronisation an allocation brings.  For them
// the per-partition maxima, exp-sums and partial outputs live in a fixed array inside this
// library's device image instead of in caller memory.
namespace {

// Every GPU that loads the library carries this array from load until process exit.
static __device__ __align__(256) unsigned char g_static_scratch[PA_STATIC_SCRATCH_BYTES];

inline size_t align256(size_t v) { return (v + 255u) & ~static_cast<size_t>(255u); }

// Device address of g_static_scratch on the current device.  In host code the array's name
// is only a handle of the host-side shadow, never a device pointer, so the address is asked
// from the runtime once per device (with that device current) and remembered.
int static_scratch_base(unsigned char **base) {
  constexpr int kMaxDevices = 64;
  static unsigned char *cache[kMaxDevices] = {};
  static bool known[kMaxDevices] = {};
  static std::mutex mu;
  int device = 0;
  PA_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return pa::fail(PA_ERR_CUDA, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(mu);
  if (!known[device]) {
    void *sym = nullptr;
    PA_CUDA_TRY(cudaGetSymbolAddress(&sym, g_static_scratch));
    if (sym == nullptr) return pa::fail(PA_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    cache[device] = static_cast<unsigned char *>(sym);
    known[device] = true;
  }
  *base = cache[device];
  return PA_OK;
}

} // namespace

extern "C" PA_API int launch_kernels_reduce_static_scratch(const pa_params *p, void *stream) {
  using namespace pa;
  if (p == nullptr) return fail(PA_ERR_BAD_ARG, "params is null");
  // A subset launch indexes the scratch rows by the sequence ids in a device array this call
  // cannot read; the array built into the library only has room for ids below num_seqs, so the
  // library refuses what it cannot bound.
  if (p->seq_indices != nullptr)
    return fail(PA_ERR_BAD_ARG, "the static-scratch entry point does not take seq_indices: scratch rows are "
                                "indexed by sequence id and the built-in array is sized from num_seqs");
  // size check next: it needs nothing from the device
  const size_t rows = static_cast<size_t>(p->num_seqs) * p->num_heads * p->max_num_partitions;
  const size_t stats_bytes = align256(rows * sizeof(float));
  const size_t partial_bytes = align256(rows * p->head_size * sizeof(__half));
  const size_t need = 2 * stats_bytes + partial_bytes;
  if (need > static_cast<size_t>(PA_STATIC_SCRATCH_BYTES))
    return fail(PA_ERR_BAD_ARG,
                "static scratch too small: num_seqs*num_heads*max_num_partitions = %zu rows need %zu bytes, "
                "the built-in array holds %zu",
                rows, need, static_cast<size_t>(PA_STATIC_SCRATCH_BYTES));
  pa_params q = *p;
  unsigned char *base = nullptr;
  if (p->num_seqs != 0) {
    if (int rc = static_scratch_base(&base)) return rc;
  } else {
    base = reinterpret_cast<unsigned char *>(static_cast<uintptr_t>(256)); // never dereferenced
  }
  // carve the array: [max_logits | exp_sums | partial outputs], each 256-byte aligned.
  // Nothing has to start at zero: the attention kernel writes every row the merge kernel
  // reads (partitions below ceil(ctx / partition_size)) and the merge reads no other row.
  q.max_logits = reinterpret_cast<float *>(base);
  q.exp_sums = reinterpret_cast<float *>(base + stats_bytes);
  q.tmp_out = base + 2 * stats_bytes;
  if (int rc = validate_params(&q, /*fp8_entry=*/false, /*needs_scratch=*/true)) return rc;
  if (q.num_seqs == 0) return PA_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int rc = dispatch_head_size<KV_F16, MODE_SPLIT>(&q, s)) return rc;
  return dispatch_merge(&q, s);
}
