// Shared host/device helpers for the h3sparse kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/h3sparse.h"

namespace h3s {

// Records the message returned by h3s_last_error() and returns `code`.
int fail(int code, const char *fmt, ...);

#define H3S_CHECK_ARG(cond, ...)                          \
  do {                                                    \
    if (!(cond)) return ::h3s::fail(H3S_EINVAL, __VA_ARGS__); \
  } while (0)

#define H3S_CHECK_CUDA(expr)                                                   \
  do {                                                                         \
    cudaError_t err__ = (expr);                                                \
    if (err__ != cudaSuccess)                                                  \
      return ::h3s::fail(H3S_ECUDA, "%s failed: %s", #expr,                    \
                         cudaGetErrorString(err__));                           \
  } while (0)

// Upper bound of every device-side wait of the kernels launched from now on
// (h3s_set_wait_budget_ns).
unsigned long long wait_budget_ns();

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- element loads: 8 consecutive channels of one row, widened to fp32 ----

template <typename T>
struct Elem;

template <>
struct Elem<float> {
  static constexpr int kDtype = H3S_F32;
  struct Raw { float4 a, b; };  // 8 elements as loaded
  __device__ static Raw load_raw(const float *p) {
    Raw r;
    r.a = __ldg(reinterpret_cast<const float4 *>(p));
    r.b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    return r;
  }
  __device__ static Raw zero_raw() { Raw r; r.a = make_float4(0.f, 0.f, 0.f, 0.f); r.b = r.a; return r; }
  __device__ static void unpack(const Raw &r, float (&v)[8]) {
    v[0] = r.a.x; v[1] = r.a.y; v[2] = r.a.z; v[3] = r.a.w;
    v[4] = r.b.x; v[5] = r.b.y; v[6] = r.b.z; v[7] = r.b.w;
  }
  __device__ static void load8(const float *p, float (&v)[8]) { unpack(load_raw(p), v); }
  __device__ static float round_trip(float x) { return x; }
};

template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kDtype = H3S_BF16;
  typedef uint4 Raw;  // 8 elements as loaded
  __device__ static Raw load_raw(const __nv_bfloat16 *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }
  __device__ static Raw zero_raw() { return make_uint4(0u, 0u, 0u, 0u); }
  __device__ static void load8(const __nv_bfloat16 *p, float (&v)[8]) { unpack(load_raw(p), v); }
  __device__ static void unpack(const Raw &raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static float round_trip(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
  }
};

template <>
struct Elem<__half> {
  static constexpr int kDtype = H3S_F16;
  typedef uint4 Raw;  // 8 elements as loaded
  __device__ static Raw load_raw(const __half *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }
  __device__ static Raw zero_raw() { return make_uint4(0u, 0u, 0u, 0u); }
  __device__ static void load8(const __half *p, float (&v)[8]) { unpack(load_raw(p), v); }
  __device__ static void unpack(const Raw &raw, float (&v)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  __device__ static float round_trip(float x) {
    return __half2float(__float2half_rn(x));
  }
};

// Correctly rounded a/b for many a and one b: with r = RN(1/b),
//   q0 = RN(a*r), e = a - b*q0 (exact in an FMA), q = RN(q0 + e*r)
// equals RN(a/b) (Markstein) unless b's significand is all ones, where RN(1/b)
// is not accurate enough; `exact` is false there and the IEEE divide is used.
struct SharedDivisor {
  float b, r;
  bool exact;
};

__device__ __forceinline__ SharedDivisor make_divisor(float divisor) {
  SharedDivisor d;
  d.b = divisor;
  d.r = __frcp_rn(divisor);
  d.exact = (__float_as_uint(divisor) & 0x007fffffu) != 0x007fffffu && fabsf(divisor) > 1.0e-30f &&
            fabsf(divisor) < 1.0e30f;
  return d;
}

// kExact is d.exact, tested ONCE by the caller around its whole element loop: with the
// test inside `divide` the compiler keeps the IEEE division sequence in the loop body
// next to the three-instruction path, which made the quantisers several times slower.
template <bool kExact>
__device__ __forceinline__ float divide(const SharedDivisor &d, float a) {
  if (!kExact) return __fdiv_rn(a, d.b);
  const float q0 = __fmul_rn(a, d.r);
  const float e = __fmaf_rn(-d.b, q0, a);
  return __fmaf_rn(e, d.r, q0);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace h3s
