// launch_kernels_reduce: fp16 KV cache, split-context decode attention
// (per-partition attention kernel + merge kernel).  Host counterpart of the
// reference's dispatch_paged_attention / launch_paged_attn_v2
// (paged_attention_reduce/launch_kernels_reduce.h:18-78,80-197).
#include "launch_common.cuh"

namespace pa {
int read_status_reduce(int *v) { return read_and_clear_device_status(v); }
} // namespace pa

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
