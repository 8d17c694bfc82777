// Status strings, version and device check of the C ABI.
#include "nvfp4_common.cuh"

namespace nvfp4 {

int check_device_sm100() {
  // -1 unknown, 0 not sm_100, 1 sm_100; indexed by device ordinal
  static int cache[64];
  static bool init = false;
  if (!init) {
    for (int& c : cache) c = -1;
    init = true;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return NVFP4_ERR_UNSUPPORTED_ARCH;
  if (dev >= 0 && dev < 64 && cache[dev] >= 0)
    return cache[dev] ? NVFP4_OK : NVFP4_ERR_UNSUPPORTED_ARCH;
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return NVFP4_ERR_UNSUPPORTED_ARCH;
  if (dev >= 0 && dev < 64) cache[dev] = (major == 10);
  return major == 10 ? NVFP4_OK : NVFP4_ERR_UNSUPPORTED_ARCH;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

}  // namespace nvfp4

extern "C" {

const char* nvfp4_status_string(int status) {
  switch (status) {
    case NVFP4_OK: return "ok";
    case NVFP4_ERR_BAD_ARG: return "bad argument";
    case NVFP4_ERR_BAD_ALIGN: return "pointer or leading dimension not 16-byte aligned";
    case NVFP4_ERR_UNSUPPORTED_ARCH: return "device is not compute capability 10.x (sm_100)";
    case NVFP4_ERR_LAUNCH_FAILED: return "kernel launch failed";
    case NVFP4_ERR_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

int nvfp4_version(void) { return 100; }

int nvfp4_init(int device, int* cc_major, int* cc_minor) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count)
    return NVFP4_ERR_UNSUPPORTED_ARCH;
  int major = 0, minor = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess)
    return NVFP4_ERR_UNSUPPORTED_ARCH;
  if (cc_major) *cc_major = major;
  if (cc_minor) *cc_minor = minor;
  return major == 10 ? NVFP4_OK : NVFP4_ERR_UNSUPPORTED_ARCH;
}

}  // extern "C"
