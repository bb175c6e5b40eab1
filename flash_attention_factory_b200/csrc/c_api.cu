// Library-wide pieces of the C ABI: error strings, device queries, the policy
// query and the lookup of the driver's tensor-map encoder.
#include <mutex>

#include "launch_common.cuh"

namespace pa {

static thread_local char g_last_error[512] = "";

void set_last_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return static_cast<EncodeTiledFn>(nullptr);
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

int get_device_info(DeviceInfo *info) {
  constexpr int kMaxDevices = 64;
  static DeviceInfo cache[kMaxDevices];
  static bool known[kMaxDevices] = {};
  static std::mutex mu;
  int device = 0;
  PA_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return fail(PA_ERR_CUDA, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(mu);
  if (!known[device]) {
    PA_CUDA_TRY(cudaDeviceGetAttribute(&cache[device].sm_count, cudaDevAttrMultiProcessorCount, device));
    PA_CUDA_TRY(cudaDeviceGetAttribute(&cache[device].cc_major, cudaDevAttrComputeCapabilityMajor, device));
    known[device] = true;
  }
  *info = cache[device];
  return PA_OK;
}

// Self-test of the bounded wait: one CTA waits on an mbarrier that nothing ever completes.
// The wait has to give up after `limit_ns`, raise the CTA's abort flag and leave the kernel
// through the normal exit, which records the time-out in the device status word.
__global__ void selftest_wait_kernel(unsigned long long limit_ns, int *gave_up) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0u;
    mbar_fence_init();
  }
  __syncthreads();
  const bool ok = mbar_wait_bounded(&bar, 0u, &abort_flag, limit_ns); // nobody arrives
  __syncthreads();
  if (threadIdx.x == 0) {
    *gave_up = ok ? 0 : 1;
    if (abort_flag != 0u) atomicExch(&g_pa_device_status, 4);
  }
}

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

PA_API const char *pa_last_error(void) { return pa::g_last_error; }

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

PA_API int pa_selftest_wait_timeout(uint32_t limit_us) {
  if (limit_us == 0 || limit_us > 500000u) return pa::fail(PA_ERR_BAD_ARG, "limit_us must be in 1..500000");
  int *flag = nullptr;
  cudaError_t err = cudaMalloc(&flag, sizeof(int));
  if (err != cudaSuccess) return pa::fail(PA_ERR_CUDA, "cudaMalloc failed: %s", cudaGetErrorString(err));
  err = cudaMemset(flag, 0xff, sizeof(int));
  if (err == cudaSuccess) {
    pa::selftest_wait_kernel<<<1, 64>>>(static_cast<unsigned long long>(limit_us) * 1000ull, flag);
    err = cudaDeviceSynchronize();
  }
  int gave_up = -1;
  if (err == cudaSuccess) err = cudaMemcpy(&gave_up, flag, sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(flag);
  if (err != cudaSuccess) return pa::fail(PA_ERR_CUDA, "self-test failed: %s", cudaGetErrorString(err));
  if (gave_up != 1) return pa::fail(PA_ERR_CUDA, "the bounded wait did not give up (flag %d)", gave_up);
  return PA_OK;
}

PA_API int pa_device_status(void) {
  cudaError_t err = cudaDeviceSynchronize();
  if (err != cudaSuccess) return pa::fail(PA_ERR_CUDA, "cudaDeviceSynchronize failed: %s", cudaGetErrorString(err));
  int (*readers[5])(int *) = {pa::read_status_loop, pa::read_status_reduce, pa::read_status_fp8_loop,
                              pa::read_status_fp8_reduce, pa::read_and_clear_device_status};
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
