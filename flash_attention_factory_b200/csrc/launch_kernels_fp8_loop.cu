// launch_kernels_fp8_loop: FP8 (e5m2 / e4m3) KV cache, single-pass decode
// attention.  Host counterpart of the reference's
// dispatch_paged_attention_fp8_loop / launch_paged_attn_fp8_loop
// (paged_attention_fp8_loop/launch_kernels_fp8_loop.h:17-56,58-175); the format
// is a run-time field here where the reference binding fixes e5m2
// (paged_attention_fp8_loop/paged_attention_fp8_loop.cpp:43).
#include "launch_common.cuh"

namespace pa {
int read_status_fp8_loop(int *v) { return read_and_clear_device_status(v); }
} // namespace pa

PA_TIMELINE_ACCESSOR(pa_debug_timeline_fp8_loop)
PA_BOUNDS_ACCESSOR(pa_debug_bounds_fp8_loop)

extern "C" PA_API int launch_kernels_fp8_loop(const pa_params *p, void *stream, float *us_out) {
  using namespace pa;
  if (int rc = validate_params(p, /*fp8_entry=*/true, /*needs_scratch=*/false)) return rc;
  if (us_out) us_out[0] = 0.f;
  if (p->num_seqs == 0) return PA_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto attn = [&] {
    return p->kv_dtype == PA_KV_FP8_E5M2 ? dispatch_head_size<KV_E5M2, MODE_LOOP>(p, s)
                                         : dispatch_head_size<KV_E4M3, MODE_LOOP>(p, s);
  };
  return run_timed(s, us_out, attn, [] { return 0; }, false);
}
