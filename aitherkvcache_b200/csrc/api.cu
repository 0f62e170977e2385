// Library-wide entry points of the C ABI (version, last error text).
#include "common.cuh"

namespace akv {
char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}
}  // namespace akv

AKV_EXPORT int akv_version(void) { return 100; }

AKV_EXPORT const char* akv_last_error(void) { return akv::error_buffer(); }

// Compute capability of the current device as major*10+minor (e.g. 100 on B200),
// or a negative value when no device is usable.
AKV_EXPORT int akv_device_arch(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  int major = 0, minor = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
  cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
  return major * 10 + minor;
}
