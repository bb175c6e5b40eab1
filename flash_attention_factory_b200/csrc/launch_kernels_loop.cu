// launch_kernels_loop: fp16 KV cache, single-pass decode attention.
// Host counterpart of the reference's dispatch_paged_attention_loop /
// launch_paged_attn_loop (paged_attention_loop/launch_kernels_loop.h:16-54,56-173).
#include "launch_common.cuh"

namespace pa {
int read_status_loop(int *v) { return read_and_clear_device_status(v); }
} // namespace pa

PA_TIMELINE_ACCESSOR(pa_debug_timeline_loop)
PA_BOUNDS_ACCESSOR(pa_debug_bounds_loop)

extern "C" PA_API int launch_kernels_loop(const pa_params *p, void *stream, float *us_out) {
  using namespace pa;
  if (int rc = validate_params(p, /*fp8_entry=*/false, /*needs_scratch=*/false)) return rc;
  if (us_out) us_out[0] = 0.f;
  if (p->num_seqs == 0) return PA_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return run_timed(
      s, us_out, [&] { return dispatch_head_size<KV_F16, MODE_LOOP>(p, s); }, [] { return 0; }, false);
}
