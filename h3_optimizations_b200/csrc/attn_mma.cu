// Block-sparse attention on the carriers with the legacy tensor path
// (mma.sync m16n8k32, s8 x s8 -> s32 and e4m3 x e4m3 -> f32).
//
// Same arithmetic contract as the tcgen05 kernel (integer running maximum,
// lazy rescale above 2^8.75, FP32 row sums of the unrounded probabilities), kept
// deliberately simple - synchronous tile loads, no pipelining - because its
// job is to cross-check the tcgen05 kernel on the device at sizes where the
// CPU checker is too slow.
//
// One CTA = one 128-row query tile of one head; 8 warps x 16 rows.
// P leaves the QK^T accumulators in the C-fragment layout; instead of
// shuffling it into the A-fragment layout, the K index of the P.V product is
// permuted consistently on both operands: A slot 4t+i of a 16-key half maps
// to key 8*(i/2) + 2t + (i%2), and the V fragment is gathered the same way.
#include <climits>

#include "common.cuh"

namespace h3s {

int check_attn_args(const int8_t *q8, const int8_t *k8, const uint8_t *v8t, const float *q_scale,
                    const float *k_scale, const float *v_scale, const int32_t *route, int route_len,
                    int q_start, int q_stop, void *out, int out_dtype, int64_t out_stride_h,
                    int64_t out_stride_s, int heads, int sequence, const char *who);

constexpr int kMmaThreads = 256;
constexpr int kKPitch = H3S_HEAD_DIM + 16;   // bytes per key row
constexpr int kVPitchT = H3S_KV_TILE + 16;   // bytes per channel row

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__device__ __forceinline__ void mma_s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_e4m3(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename OutT> __device__ __forceinline__ void store2(OutT *dst, float a, float b);
template <> __device__ __forceinline__ void store2<float>(float *dst, float a, float b) {
  *reinterpret_cast<float2 *>(dst) = make_float2(a, b);
}
template <> __device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16 *dst, float a, float b) {
  *reinterpret_cast<__nv_bfloat162 *>(dst) = __floats2bfloat162_rn(a, b);
}
template <> __device__ __forceinline__ void store2<__half>(__half *dst, float a, float b) {
  *reinterpret_cast<__half2 *>(dst) = __floats2half2_rn(a, b);
}

template <typename OutT, bool kSplitP>
__global__ void __launch_bounds__(kMmaThreads)
sparse_attn_mma_kernel(const int8_t *__restrict__ q8, const int8_t *__restrict__ k8,
                       const uint8_t *__restrict__ v8t, const float *__restrict__ q_scale,
                       const float *__restrict__ k_scale, const float *__restrict__ v_scale,
                       const int32_t *__restrict__ route, int route_len, int q_start, int q_stop,
                       OutT *__restrict__ out, int64_t out_stride_h, int64_t out_stride_s, int heads,
                       int sequence, int q_tiles, int kv_tiles, int padded) {
  __shared__ __align__(16) unsigned char s_k[H3S_KV_TILE * kKPitch];
  __shared__ __align__(16) unsigned char s_v[H3S_HEAD_DIM * kVPitchT];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  const int n_sparse = route != nullptr ? q_stop - q_start : 0;
  const int n_dense = q_tiles - n_sparse;
  int head, tq;
  bool dense;
  {
    const int w = blockIdx.x;
    const int dense_items = heads * n_dense;
    if (w < dense_items) {
      dense = true;
      head = w / n_dense;
      const int i = w - head * n_dense;
      tq = (n_sparse == 0 || i < q_start) ? i : q_stop + (i - q_start);
    } else {
      dense = false;
      const int v = w - dense_items;
      head = v / n_sparse;
      tq = q_start + (v - head * n_sparse);
    }
  }
  const int n_iter = dense ? kv_tiles : route_len;
  const int32_t *route_row =
      dense ? nullptr : route + (static_cast<int64_t>(head) * n_sparse + (tq - q_start)) * route_len;

  // Q fragments straight from global memory (rows beyond the sequence read as zero)
  const int row_lo = tq * H3S_Q_TILE + warp * 16 + g;
  const int row_hi = row_lo + 8;
  uint32_t qa[4][4];
  {
    const int8_t *qh = q8 + static_cast<int64_t>(head) * sequence * H3S_HEAD_DIM;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int col = 32 * kk + 4 * t;
      qa[kk][0] = row_lo < sequence ? *reinterpret_cast<const uint32_t *>(qh + static_cast<int64_t>(row_lo) * H3S_HEAD_DIM + col) : 0u;
      qa[kk][1] = row_hi < sequence ? *reinterpret_cast<const uint32_t *>(qh + static_cast<int64_t>(row_hi) * H3S_HEAD_DIM + col) : 0u;
      qa[kk][2] = row_lo < sequence ? *reinterpret_cast<const uint32_t *>(qh + static_cast<int64_t>(row_lo) * H3S_HEAD_DIM + col + 16) : 0u;
      qa[kk][3] = row_hi < sequence ? *reinterpret_cast<const uint32_t *>(qh + static_cast<int64_t>(row_hi) * H3S_HEAD_DIM + col + 16) : 0u;
    }
  }
  const float qs = __ldg(q_scale + head * q_tiles + tq) * (0.08838834764831845f * 1.4426950408889634f);

  float oacc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[i][e] = 0.f;
  float m_used[2] = {-INFINITY, -INFINITY};
  float l_part[2] = {0.f, 0.f};

  const int8_t *kh = k8 + static_cast<int64_t>(head) * sequence * H3S_HEAD_DIM;
  const uint8_t *vh = v8t + static_cast<int64_t>(head) * H3S_HEAD_DIM * padded;

  for (int j = 0; j < n_iter; ++j) {
    const int tile = dense ? j : __ldg(route_row + j);
    __syncthreads();  // previous tile fully consumed
#pragma unroll
    for (int c = threadIdx.x; c < H3S_KV_TILE * 8; c += kMmaThreads) {
      const int r = c >> 3, ch = c & 7;
      const int key = tile * H3S_KV_TILE + r;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (key < sequence) v = __ldg(reinterpret_cast<const uint4 *>(kh + static_cast<int64_t>(key) * H3S_HEAD_DIM + ch * 16));
      *reinterpret_cast<uint4 *>(s_k + r * kKPitch + ch * 16) = v;
    }
#pragma unroll
    for (int c = threadIdx.x; c < H3S_HEAD_DIM * 4; c += kMmaThreads) {
      const int d = c >> 2, ch = c & 3;
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(vh + static_cast<int64_t>(d) * padded + tile * H3S_KV_TILE + ch * 16));
      *reinterpret_cast<uint4 *>(s_v + d * kVPitchT + ch * 16) = v;
    }
    __syncthreads();

    // ---- S = Q K^T ----
    int sacc[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) sacc[nb][e] = 0;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const unsigned char *kp = s_k + (8 * nb + g) * kKPitch + 32 * kk + 4 * t;
        mma_s8(sacc[nb], qa[kk], *reinterpret_cast<const uint32_t *>(kp),
               *reinterpret_cast<const uint32_t *>(kp + 16));
      }
    }

    // ---- online softmax ----
    const float c = qs * __ldg(k_scale + static_cast<int64_t>(head) * kv_tiles + tile);
    const int n_valid = min(H3S_KV_TILE, sequence - tile * H3S_KV_TILE);
    int imax[2] = {INT_MIN, INT_MIN};
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = 8 * nb + 2 * t + (e & 1);
        if (col < n_valid) imax[e >> 1] = max(imax[e >> 1], sacc[nb][e]);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      imax[h] = max(imax[h], __shfl_xor_sync(0xffffffffu, imax[h], 1));
      imax[h] = max(imax[h], __shfl_xor_sync(0xffffffffu, imax[h], 2));
      const float mx = c * static_cast<float>(imax[h]);
      if (mx > m_used[h] + 8.75f) {
        const float m_new = ceilf(mx) - 7.0f;  // largest P in (64,128]; room to 2^8.75 before the next rescale
        const float alpha = ex2(m_used[h] - m_new);
        m_used[h] = m_new;
        l_part[h] *= alpha;
#pragma unroll
        for (int db = 0; db < 16; ++db) {
          oacc[db][2 * h] *= alpha;
          oacc[db][2 * h + 1] *= alpha;
        }
      }
    }
    float p[8][4];
    float r[kSplitP ? 8 : 1][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = 8 * nb + 2 * t + (e & 1);
        float v = ex2(fmaf(c, static_cast<float>(sacc[nb][e]), -m_used[e >> 1]));
        if (col >= n_valid) v = 0.f;
        l_part[e >> 1] += v;
        if (kSplitP) {
          const float hi = __uint_as_float(__float_as_uint(v) & 0xfff00000u);  // 4 significant bits, exact in E4M3
          r[nb][e] = v - hi;
          v = hi;
        }
        p[nb][e] = v;
      }
    }

    // ---- O += P V (key index permuted identically on both operands) ----
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t pa[4];
      pa[0] = e4m3x4(p[4 * ks + 0][0], p[4 * ks + 0][1], p[4 * ks + 1][0], p[4 * ks + 1][1]);
      pa[1] = e4m3x4(p[4 * ks + 0][2], p[4 * ks + 0][3], p[4 * ks + 1][2], p[4 * ks + 1][3]);
      pa[2] = e4m3x4(p[4 * ks + 2][0], p[4 * ks + 2][1], p[4 * ks + 3][0], p[4 * ks + 3][1]);
      pa[3] = e4m3x4(p[4 * ks + 2][2], p[4 * ks + 2][3], p[4 * ks + 3][2], p[4 * ks + 3][3]);
      uint32_t pl[4] = {0u, 0u, 0u, 0u};
      if (kSplitP) {
        pl[0] = e4m3x4(r[4 * ks + 0][0], r[4 * ks + 0][1], r[4 * ks + 1][0], r[4 * ks + 1][1]);
        pl[1] = e4m3x4(r[4 * ks + 0][2], r[4 * ks + 0][3], r[4 * ks + 1][2], r[4 * ks + 1][3]);
        pl[2] = e4m3x4(r[4 * ks + 2][0], r[4 * ks + 2][1], r[4 * ks + 3][0], r[4 * ks + 3][1]);
        pl[3] = e4m3x4(r[4 * ks + 2][2], r[4 * ks + 2][3], r[4 * ks + 3][2], r[4 * ks + 3][3]);
      }
#pragma unroll
      for (int db = 0; db < 16; ++db) {
        const unsigned char *vp = s_v + (8 * db + g) * kVPitchT + 32 * ks + 2 * t;
        const uint32_t b0 = static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(vp)) |
                            (static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(vp + 8)) << 16);
        const uint32_t b1 = static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(vp + 16)) |
                            (static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(vp + 24)) << 16);
        mma_e4m3(oacc[db], pa, b0, b1);
        if (kSplitP) mma_e4m3(oacc[db], pl, b0, b1);
      }
    }
  }

  // ---- epilogue ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_part[h] += __shfl_xor_sync(0xffffffffu, l_part[h], 1);
    l_part[h] += __shfl_xor_sync(0xffffffffu, l_part[h], 2);
  }
  const float inv_l[2] = {1.0f / l_part[0], 1.0f / l_part[1]};
  const float *vs = v_scale + head * H3S_HEAD_DIM;
#pragma unroll
  for (int db = 0; db < 16; ++db) {
    const int d = 8 * db + 2 * t;
    const float s0 = __ldg(vs + d), s1 = __ldg(vs + d + 1);
    if (row_lo < sequence)
      store2<OutT>(out + head * out_stride_h + static_cast<int64_t>(row_lo) * out_stride_s + d,
                   oacc[db][0] * s0 * inv_l[0], oacc[db][1] * s1 * inv_l[0]);
    if (row_hi < sequence)
      store2<OutT>(out + head * out_stride_h + static_cast<int64_t>(row_hi) * out_stride_s + d,
                   oacc[db][2] * s0 * inv_l[1], oacc[db][3] * s1 * inv_l[1]);
  }
}

template <typename OutT>
static int launch_attn_mma(const int8_t *q8, const int8_t *k8, const uint8_t *v8t, const float *q_scale,
                           const float *k_scale, const float *v_scale, const int32_t *route, int route_len,
                           int q_start, int q_stop, void *out, int64_t osh, int64_t oss, int heads,
                           int sequence, bool split_p, cudaStream_t stream) {
  const int q_tiles = ceil_div(sequence, H3S_Q_TILE), kv_tiles = ceil_div(sequence, H3S_KV_TILE);
  const int padded = ceil_div(sequence, 128) * 128;
  if (split_p) {
    sparse_attn_mma_kernel<OutT, true><<<heads * q_tiles, kMmaThreads, 0, stream>>>(
        q8, k8, v8t, q_scale, k_scale, v_scale, route, route_len, q_start, q_stop, static_cast<OutT *>(out),
        osh, oss, heads, sequence, q_tiles, kv_tiles, padded);
  } else {
    sparse_attn_mma_kernel<OutT, false><<<heads * q_tiles, kMmaThreads, 0, stream>>>(
        q8, k8, v8t, q_scale, k_scale, v_scale, route, route_len, q_start, q_stop, static_cast<OutT *>(out),
        osh, oss, heads, sequence, q_tiles, kv_tiles, padded);
  }
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

}  // namespace h3s

extern "C" int h3s_sparse_attn_fwd_mma(const int8_t *q8, const int8_t *k8, const uint8_t *v8t,
                                       const float *q_scale, const float *k_scale, const float *v_scale,
                                       const int32_t *route, int route_len, int q_start, int q_stop,
                                       void *out, int out_dtype, int64_t out_stride_h,
                                       int64_t out_stride_s, int heads, int sequence, int flags,
                                       h3s_stream_t stream) {
  using namespace h3s;
  {
    int rc = check_attn_args(q8, k8, v8t, q_scale, k_scale, v_scale, route, route_len, q_start, q_stop, out,
                             out_dtype, out_stride_h, out_stride_s, heads, sequence, "sparse_attn_fwd_mma");
    if (rc) return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool sp = (flags & H3S_ATTN_P_SINGLE) == 0;
  switch (out_dtype) {
    case H3S_F32: return launch_attn_mma<float>(q8, k8, v8t, q_scale, k_scale, v_scale, route, route_len, q_start, q_stop, out, out_stride_h, out_stride_s, heads, sequence, sp, s);
    case H3S_BF16: return launch_attn_mma<__nv_bfloat16>(q8, k8, v8t, q_scale, k_scale, v_scale, route, route_len, q_start, q_stop, out, out_stride_h, out_stride_s, heads, sequence, sp, s);
    default: return launch_attn_mma<__half>(q8, k8, v8t, q_scale, k_scale, v_scale, route, route_len, q_start, q_stop, out, out_stride_h, out_stride_s, heads, sequence, sp, s);
  }
}
