// Library-level entry points: error text, ABI version, device capability.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace h3s {

static thread_local char g_error[512] = "";

int fail(int code, const char *fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

}  // namespace h3s

extern "C" {

int h3s_abi_version(void) { return 1; }

const char *h3s_last_error(void) { return h3s::g_error; }

int h3s_device_capability(void) {
  int device = 0, major = 0, minor = 0;
  H3S_CHECK_CUDA(cudaGetDevice(&device));
  H3S_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  H3S_CHECK_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  return major * 10 + minor;
}

}  // extern "C"
