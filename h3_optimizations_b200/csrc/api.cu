// Library-level entry points: error text, ABI version, device capability.
#include <atomic>
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

static std::atomic<unsigned long long> g_wait_budget_ns{2000000000ull};

unsigned long long wait_budget_ns() { return g_wait_budget_ns.load(std::memory_order_relaxed); }

}  // namespace h3s

extern "C" {

int h3s_abi_version(void) { return 1; }

int h3s_set_wait_budget_ns(unsigned long long nanoseconds) {
  H3S_CHECK_ARG(nanoseconds >= 1000ull && nanoseconds <= 60000000000ull,
                "set_wait_budget_ns: %llu ns is outside [1 us, 60 s]", nanoseconds);
  h3s::g_wait_budget_ns.store(nanoseconds, std::memory_order_relaxed);
  return H3S_OK;
}

unsigned long long h3s_get_wait_budget_ns(void) { return h3s::wait_budget_ns(); }

const char *h3s_last_error(void) { return h3s::g_error; }

int h3s_device_capability(void) {
  int device = 0, major = 0, minor = 0;
  H3S_CHECK_CUDA(cudaGetDevice(&device));
  H3S_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  H3S_CHECK_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  return major * 10 + minor;
}

}  // extern "C"
