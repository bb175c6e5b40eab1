// Host pieces every library of this package links: the per-thread error string, the lookup of
// the driver's tensor-map encoder and the cached device properties.
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

const char *last_error() { return g_last_error; }

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

} // namespace pa
