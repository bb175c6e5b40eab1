// Test and measurement aids, built into a library of their own
// (libpaged_attention_b200_test_aids.so) so that the product library stays free of code that
// allocates device memory: a self-test of the bounded mbarrier wait and a read-only streaming
// probe.  Both use the product's own device helpers (include/paged_attention_utils.hpp) and
// status-word code (launch_common.cuh), compiled into this library a second time.
#include "launch_common.cuh"
#include "paged_attention_b200_test_aids.h"

namespace pa {

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

// Read-only streaming probe, method 0: every thread pulls 16-byte words with a grid stride,
// eight loads in flight, and folds them into a checksum that is stored once per launch only for
// a value no real buffer produces in practice, so the loads cannot be optimised away and
// nothing is written.
__device__ __forceinline__ void stream_fold(uint4 &acc, const uint4 &v) {
  acc.x ^= v.x;
  acc.y += v.y;
  acc.z ^= v.z;
  acc.w += v.w;
}

__device__ __forceinline__ void stream_read_range(const uint4 *__restrict__ src, unsigned long long n16, uint4 &acc) {
  const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * blockDim.x;
  unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + 7ull * stride < n16; i += 8ull * stride) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcs(src + i + static_cast<unsigned long long>(u) * stride);
#pragma unroll
    for (int u = 0; u < 8; ++u) stream_fold(acc, v[u]);
  }
  for (; i < n16; i += stride) stream_fold(acc, __ldcs(src + i));
}

__global__ void __launch_bounds__(512)
stream_read_kernel(const uint4 *__restrict__ a, unsigned long long na16, const uint4 *__restrict__ b,
                   unsigned long long nb16, unsigned *sink) {
  uint4 acc = make_uint4(0u, 0u, 0u, 0u);
  stream_read_range(a, na16, acc);
  if (nb16 != 0) stream_read_range(b, nb16, acc);
  if ((acc.x ^ acc.y) == 0x9e3779b9u && (acc.z ^ acc.w) == 0x7f4a7c15u) *sink = acc.x;
}

// Method 1, the same measurement with the copy engine the attention kernels use: one thread
// per CTA keeps a ring of bulk copies into shared memory in flight and never looks at the
// data.  Chunks are dealt round-robin over the grid; every wait is bounded.
constexpr uint32_t kProbeChunk = 16384, kProbeStages = 6;

__global__ void __launch_bounds__(32)
stream_read_bulk_kernel(const unsigned char *__restrict__ a, unsigned long long chunks_a,
                        const unsigned char *__restrict__ b, unsigned long long chunks_b, int *gave_up) {
  extern __shared__ __align__(1024) unsigned char probe_ring[];
  __shared__ uint64_t bar[kProbeStages];
  __shared__ uint32_t abort_flag;
  if (threadIdx.x != 0) return;
  for (uint32_t s = 0; s < kProbeStages; ++s) mbar_init(&bar[s], 1);
  abort_flag = 0u;
  mbar_fence_init();
  const uint64_t policy = l2_evict_first_policy();
  const uint32_t ring = smem_u32(probe_ring);
  const unsigned long long total = chunks_a + chunks_b;
  unsigned long long issued = 0;
  bool ok = true;
  for (unsigned long long c = blockIdx.x; c < total; c += gridDim.x, ++issued) {
    const uint32_t stage = static_cast<uint32_t>(issued % kProbeStages);
    const unsigned long long use = issued / kProbeStages;
    if (use > 0) ok = mbar_wait_bounded(&bar[stage], static_cast<uint32_t>((use - 1) & 1ull), &abort_flag);
    if (!ok) break;
    const unsigned char *src = (c < chunks_a) ? a + c * kProbeChunk : b + (c - chunks_a) * kProbeChunk;
    mbar_arrive_expect_tx(&bar[stage], kProbeChunk);
    bulk_load_1d(ring + stage * kProbeChunk, src, kProbeChunk, &bar[stage], policy);
  }
  // drain: the last copy into every stage that was used has to land before the CTA exits
  for (uint32_t s = 0; s < kProbeStages && s < issued; ++s) {
    const unsigned long long uses = (issued - s + kProbeStages - 1) / kProbeStages; // copies issued into stage s
    if (!mbar_wait_bounded(&bar[s], static_cast<uint32_t>((uses - 1) & 1ull), &abort_flag)) ok = false;
  }
  if (!ok) {
    *gave_up = 1;
    atomicExch(&g_pa_device_status, 4);
  }
}

} // namespace pa

extern "C" {

PA_API const char *pa_aid_last_error(void) { return pa::last_error(); }

PA_API int pa_aid_selftest_wait_timeout(uint32_t limit_us, int32_t *status_word) {
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
  // the status word of this translation unit, read and cleared by the function the product's
  // pa_device_status() applies to each of its own units
  int word = 0;
  if (int rc = pa::read_and_clear_device_status(&word)) return rc;
  if (status_word != nullptr) *status_word = word;
  return PA_OK;
}

PA_API int pa_aid_measure_read_bandwidth(const void *buf, uint64_t bytes, const void *buf2, uint64_t bytes2,
                                     uint32_t method, uint32_t iters, void *stream, float *gb_per_s) {
  if (buf == nullptr || gb_per_s == nullptr) return pa::fail(PA_ERR_BAD_ARG, "buf or gb_per_s is null");
  if (buf2 == nullptr) bytes2 = 0;
  if (((reinterpret_cast<uintptr_t>(buf) | reinterpret_cast<uintptr_t>(buf2)) & 15u) != 0 ||
      bytes < pa::kProbeChunk || iters == 0 || iters > 1000u || method > 1u)
    return pa::fail(PA_ERR_BAD_ARG, "buffers must be 16-byte aligned, bytes >= 16384, iters in 1..1000, method 0 or 1");
  pa::DeviceInfo dev;
  if (int rc = pa::get_device_info(&dev)) return rc;
  int *flag = nullptr; // checksum sink of method 0, gave-up flag of method 1; stays 0 in both
  cudaError_t err = cudaMalloc(&flag, sizeof(int));
  if (err == cudaSuccess) err = cudaMemset(flag, 0, sizeof(int));
  constexpr uint32_t ring_bytes = pa::kProbeChunk * pa::kProbeStages;
  if (err == cudaSuccess && method == 1u)
    err = cudaFuncSetAttribute(pa::stream_read_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(ring_bytes));
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  if (err == cudaSuccess) err = cudaEventCreate(&t0);
  if (err == cudaSuccess) err = cudaEventCreate(&t1);
  if (err != cudaSuccess) {
    if (t0) cudaEventDestroy(t0);
    cudaFree(flag);
    return pa::fail(PA_ERR_CUDA, "read probe set-up failed: %s", cudaGetErrorString(err));
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned long long unit = (method == 0u) ? 16ull : pa::kProbeChunk;
  const unsigned long long na = bytes / unit, nb = bytes2 / unit;
  auto launch = [&]() {
    if (method == 0u)
      pa::stream_read_kernel<<<static_cast<unsigned>(dev.sm_count) * 4u, 512, 0, st>>>(
          static_cast<const uint4 *>(buf), na, static_cast<const uint4 *>(buf2), nb,
          reinterpret_cast<unsigned *>(flag));
    else
      pa::stream_read_bulk_kernel<<<static_cast<unsigned>(dev.sm_count) * 2u, 32, ring_bytes, st>>>(
          static_cast<const unsigned char *>(buf), na, static_cast<const unsigned char *>(buf2), nb, flag);
  };
  float ms = 0.f;
  launch(); // warm-up
  cudaEventRecord(t0, st);
  for (uint32_t k = 0; k < iters; ++k) launch();
  cudaEventRecord(t1, st);
  err = cudaEventSynchronize(t1);
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, t0, t1);
  int gave_up = 0;
  if (err == cudaSuccess && method == 1u) err = cudaMemcpy(&gave_up, flag, sizeof(int), cudaMemcpyDeviceToHost);
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  cudaFree(flag);
  if (err != cudaSuccess) return pa::fail(PA_ERR_CUDA, "read probe failed: %s", cudaGetErrorString(err));
  if (gave_up != 0) return pa::fail(PA_ERR_TIMEOUT, "the read probe gave up a bounded wait on an mbarrier");
  *gb_per_s = (ms > 0.f) ? static_cast<float>(static_cast<double>((na + nb) * unit) * iters / (ms * 1e-3) / 1e9) : 0.f;
  return PA_OK;
}

PA_API int pa_aid_time_launches(pa_aid_launch_fn launch, const pa_params *params, uint32_t num_params,
                                uint32_t calls, void *stream, float *us_per_call) {
  if (launch == nullptr || params == nullptr || num_params == 0 || calls == 0 || us_per_call == nullptr)
    return pa::fail(PA_ERR_BAD_ARG, "time_launches: null argument or zero count");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  PA_CUDA_TRY(cudaEventCreate(&t0));
  PA_CUDA_TRY(cudaEventCreate(&t1));
  int rc = PA_OK;
  cudaError_t err = cudaEventRecord(t0, st);
  for (uint32_t i = 0; i < calls && rc == PA_OK && err == cudaSuccess; ++i)
    rc = launch(params + (i % num_params), stream, nullptr);
  if (rc == PA_OK && err == cudaSuccess) err = cudaEventRecord(t1, st);
  if (rc == PA_OK && err == cudaSuccess) err = cudaEventSynchronize(t1);
  float ms = 0.f;
  if (rc == PA_OK && err == cudaSuccess) err = cudaEventElapsedTime(&ms, t0, t1);
  cudaEventDestroy(t0);
  cudaEventDestroy(t1);
  if (rc != PA_OK) return pa::fail(rc, "time_launches: the launcher returned %d", rc);
  if (err != cudaSuccess) return pa::fail(PA_ERR_CUDA, "time_launches: %s", cudaGetErrorString(err));
  *us_per_call = ms * 1000.f / static_cast<float>(calls);
  return PA_OK;
}

} // extern "C"
