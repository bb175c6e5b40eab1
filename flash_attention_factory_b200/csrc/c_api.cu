// Library-wide pieces of the C ABI: the policy query, the host-buffer decode step and the
// device status word.
#include "launch_common.cuh"

namespace pa {

int read_status_loop(int *v);
int read_status_reduce(int *v);
int read_status_fp8_loop(int *v);
int read_status_fp8_reduce(int *v);

} // namespace pa

template <int D>
static void fill_policy(pa_policy_info *info) {
  using P16 = pa::paged_attention_policy_v2<D, pa::KV_F16>;
  using P8 = pa::paged_attention_policy_v2<D, pa::KV_E5M2>;
  info->partition_size = P16::partition_size;
  info->stages = P16::stages;
  info->head_size_stride = P16::head_size_stride;
  info->partition_stride = P16::partition_stride;
  info->max_partitions_per_sg = P16::max_partitions_per_sg;
  info->tokens_per_stage = P16::tokens_per_stage;
  info->ring_stages = P16::ring_stages;
  info->ring_stages_fp8 = P8::ring_stages;
  info->consumer_warps = P16::consumer_warps;
  info->threads_per_cta = P16::threads_per_cta;
}

extern "C" {

PA_API const char *pa_last_error(void) { return pa::last_error(); }

PA_API const char *pa_version(void) { return "0.1"; }

PA_API uint32_t pa_partition_size(uint32_t head_size) {
  if (head_size == 128) return pa::paged_attention_policy_v2<128, pa::KV_F16>::partition_size;
  if (head_size == 64) return pa::paged_attention_policy_v2<64, pa::KV_F16>::partition_size;
  return 0;
}

PA_API int pa_query_policy(uint32_t head_size, uint32_t block_size, uint32_t group, pa_policy_info *info) {
  if (info == nullptr) return pa::fail(PA_ERR_BAD_ARG, "info is null");
  const bool block_ok = block_size == 16 || block_size == 32 || block_size == 64 || block_size == 128;
  if ((head_size != 128 && head_size != 64) || !block_ok)
    return pa::fail(PA_ERR_UNSUPPORTED, "Unsupported head size or block size");
  if (group < 1 || group > 8) return pa::fail(PA_ERR_UNSUPPORTED, "Unsupported number of queries per token");
  if (head_size == 128) fill_policy<128>(info);
  else fill_policy<64>(info);
  return PA_OK;
}

PA_API int pa_device_status(void) {
  cudaError_t err = cudaDeviceSynchronize();
  if (err != cudaSuccess) return pa::fail(PA_ERR_CUDA, "cudaDeviceSynchronize failed: %s", cudaGetErrorString(err));
  int (*readers[4])(int *) = {pa::read_status_loop, pa::read_status_reduce, pa::read_status_fp8_loop,
                              pa::read_status_fp8_reduce};
  int worst = 0;
  for (auto reader : readers) {
    int v = 0;
    if (int rc = reader(&v)) return rc;
    if (v != 0) worst = v;
  }
  if (worst != 0) return pa::fail(PA_ERR_TIMEOUT, "a kernel gave up a bounded wait on an mbarrier");
  return PA_OK;
}

} // extern "C"
