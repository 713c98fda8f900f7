// Host-side plumbing shared by the C ABI entry points.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>
#include <mutex>

namespace cutb {

static thread_local char g_last_error[512] = "";

void set_last_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

const char *last_error() { return g_last_error; }

int cuda_fail(cudaError_t e, const char *what) {
  set_last_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return CUTB_ERR_CUDA;
}

int get_device_info(DeviceInfo *out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) {
    set_last_error("device index %d out of range", dev);
    return CUTB_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev].device != dev) {
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
    cache[dev].device = dev;
    cache[dev].sm_count = prop.multiProcessorCount;
    cache[dev].cc_major = prop.major;
    cache[dev].cc_minor = prop.minor;
    cache[dev].smem_optin = prop.sharedMemPerBlockOptin;
    cache[dev].smem_per_sm = prop.sharedMemPerMultiprocessor;
  }
  *out = cache[dev];
  return CUTB_OK;
}

}  // namespace cutb
