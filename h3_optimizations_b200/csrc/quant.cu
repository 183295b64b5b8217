// Carrier quantisation kernels (HBM-bound): whole-sequence column statistics,
// per-block INT8 Q/K with tile means, FP8-E4M3 transposed V.
//
// Thread mapping shared by all three: 16 consecutive threads read one
// 128-channel row as 16-byte vectors (8 channels each), so a warp covers two
// full rows and every global load/store is a fully used 128/256/512-byte line.
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace h3s {

// ---------------------------------------------------------------------------
// Column statistics: sum_s K[h,s,d] (FP64) and max_s |V[h,s,d]|.
// scratch layout: double k_sum[heads*128]; uint32 v_amax_bits[heads*128].
// ---------------------------------------------------------------------------

constexpr int kStatsThreads = 256;
constexpr int kStatsRowsPerBlock = 512;

template <typename T>
__global__ void __launch_bounds__(kStatsThreads)
column_stats_kernel(const T *__restrict__ k, int64_t k_stride_h, int64_t k_stride_s,
                    const T *__restrict__ v, int64_t v_stride_h, int64_t v_stride_s,
                    int sequence, double *__restrict__ k_sum,
                    unsigned int *__restrict__ v_amax_bits) {
  __shared__ double red[kStatsThreads / 16][H3S_HEAD_DIM];
  const int head = blockIdx.y;
  const bool is_v = blockIdx.z == 1;
  const T *src = is_v ? v : k;
  if (src == nullptr) return;
  const int64_t stride_h = is_v ? v_stride_h : k_stride_h;
  const int64_t stride_s = is_v ? v_stride_s : k_stride_s;
  const int slot = threadIdx.x >> 4;
  const int c0 = (threadIdx.x & 15) * 8;
  const int row_begin = blockIdx.x * kStatsRowsPerBlock;
  const int row_end = min(row_begin + kStatsRowsPerBlock, sequence);
  double acc[8];
  float amax[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { acc[i] = 0.0; amax[i] = 0.f; }
  const T *base = src + head * stride_h + c0;
  for (int row = row_begin + slot; row < row_end; row += kStatsThreads / 16) {
    float x[8];
    Elem<T>::load8(base + row * stride_s, x);
    if (is_v) {
#pragma unroll
      for (int i = 0; i < 8; ++i) amax[i] = fmaxf(amax[i], fabsf(x[i]));
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += static_cast<double>(x[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[slot][c0 + i] = is_v ? static_cast<double>(amax[i]) : acc[i];
  __syncthreads();
  if (threadIdx.x < H3S_HEAD_DIM) {
    const int d = threadIdx.x;
    if (is_v) {
      double m = 0.0;
#pragma unroll
      for (int s = 0; s < kStatsThreads / 16; ++s) m = fmax(m, red[s][d]);
      // non-negative floats order like their bit patterns
      atomicMax(&v_amax_bits[head * H3S_HEAD_DIM + d], __float_as_uint(static_cast<float>(m)));
    } else {
      double s = 0.0;
#pragma unroll
      for (int i = 0; i < kStatsThreads / 16; ++i) s += red[i][d];
      atomicAdd(&k_sum[head * H3S_HEAD_DIM + d], s);
    }
  }
}

template <typename T>
__global__ void column_stats_finalize_kernel(const double *__restrict__ k_sum,
                                             const unsigned int *__restrict__ v_amax_bits,
                                             int total, int sequence, float v_bound,
                                             float *__restrict__ k_mean,
                                             float *__restrict__ v_scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  if (k_mean != nullptr) {
    const float mean = static_cast<float>(k_sum[i] / static_cast<double>(sequence));
    k_mean[i] = Elem<T>::round_trip(mean);
  }
  if (v_scale != nullptr) {
    const float amax = __uint_as_float(v_amax_bits[i]);
    v_scale[i] = fmaxf(__fdiv_rn(amax, v_bound), 1.0e-20f);
  }
}

// ---------------------------------------------------------------------------
// Per-block INT8 quantisation with optional tile means.
// One CTA = one (block, head); the whole block lives in registers, as loaded
// (64 values per thread, 32 registers for 16-bit inputs), between the amax
// reduction and the store, so it is read from memory exactly once.
// ---------------------------------------------------------------------------

template <typename T, int BLOCK, bool kHasMean>
__global__ void __launch_bounds__(BLOCK * 2, (sizeof(T) == 2 ? 1024 : 512) / (BLOCK * 2))
quant_qk_blocks_kernel(const T *__restrict__ x, int64_t stride_h, int64_t stride_s,
                       const float *__restrict__ mean, int8_t *__restrict__ out,
                       float *__restrict__ scale_out, void *__restrict__ summary,
                       int summary_dtype, int rows, int row_start, int sequence_total,
                       int blocks_total) {
  constexpr int kThreads = BLOCK * 2;
  constexpr int kSlots = kThreads / 16;  // rows per pass
  constexpr int kPasses = BLOCK / kSlots;  // == 8
  __shared__ float warp_amax[kThreads / 32];
  __shared__ double red[kSlots][H3S_HEAD_DIM];

  const int local_block = blockIdx.x;
  const int head = blockIdx.y;
  const int slot = threadIdx.x >> 4;
  const int c0 = (threadIdx.x & 15) * 8;
  const int first_row = local_block * BLOCK;  // within this chunk
  const int valid_rows = min(BLOCK, rows - first_row);

  float mu[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mu[i] = 0.f;
  if (kHasMean) {
#pragma unroll
    for (int i = 0; i < 8; ++i) mu[i] = __ldg(mean + head * H3S_HEAD_DIM + c0 + i);
  }

  typename Elem<T>::Raw raw[kPasses];
  float col[8];  // this thread's rows (at most 8) summed in fp32, widened once
#pragma unroll
  for (int i = 0; i < 8; ++i) col[i] = 0.f;
  float amax = 0.f;
  const T *base = x + head * stride_h + c0;
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const int r = p * kSlots + slot;
    raw[p] = r < valid_rows ? Elem<T>::load_raw(base + static_cast<int64_t>(first_row + r) * stride_s)
                            : Elem<T>::zero_raw();
  }
#pragma unroll
  for (int p = 0; p < kPasses; ++p) {
    const int r = p * kSlots + slot;
    if (r < valid_rows) {
      float v[8];
      Elem<T>::unpack(raw[p], v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        col[i] = __fadd_rn(col[i], v[i]);
        amax = fmaxf(amax, fabsf(kHasMean ? __fsub_rn(v[i], mu[i]) : v[i]));
      }
    }
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) warp_amax[threadIdx.x >> 5] = amax;
  if (summary != nullptr) {
#pragma unroll
    for (int i = 0; i < 8; ++i) red[slot][c0 + i] = static_cast<double>(col[i]);
  }
  __syncthreads();
  amax = warp_amax[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) amax = fmaxf(amax, warp_amax[w]);
  const float scale = __fadd_rn(__fdiv_rn(amax, 127.0f), 1.0e-7f);
  const SharedDivisor by_scale = make_divisor(scale);

  const int global_block = row_start / BLOCK + local_block;
  if (threadIdx.x == 0 && scale_out != nullptr) scale_out[head * blocks_total + global_block] = scale;

  int8_t *dst = out + (static_cast<int64_t>(head) * sequence_total + row_start + first_row) *
                          H3S_HEAD_DIM + c0;
  // code = trunc(v/scale +- 0.5): the half carries the quotient's sign bit, the four
  // codes of a word are gathered with byte permutes.  The divisor's exactness is
  // tested once, around the whole loop (see divide<>).
  auto emit = [&](auto exact_tag) {
    constexpr bool kExact = decltype(exact_tag)::value;
#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      const int r = p * kSlots + slot;
      if (out != nullptr && r < valid_rows) {
        float v[8];
        Elem<T>::unpack(raw[p], v);
        uint32_t code[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float q = divide<kExact>(by_scale, kHasMean ? __fsub_rn(v[i], mu[i]) : v[i]);
          const float half = __uint_as_float((__float_as_uint(q) & 0x80000000u) | 0x3f000000u);
          q = __fadd_rn(q, half);
          code[i] = static_cast<uint32_t>(static_cast<int>(q));  // truncation toward zero
        }
        uint32_t packed[2];
#pragma unroll
        for (int w = 0; w < 2; ++w)
          packed[w] = __byte_perm(__byte_perm(code[4 * w], code[4 * w + 1], 0x0040),
                                  __byte_perm(code[4 * w + 2], code[4 * w + 3], 0x0040), 0x5410);
        *reinterpret_cast<uint2 *>(dst + static_cast<int64_t>(r) * H3S_HEAD_DIM) =
            make_uint2(packed[0], packed[1]);
      }
    }
  };
  if (by_scale.exact) emit(std::true_type{}); else emit(std::false_type{});

  if (summary != nullptr && threadIdx.x < H3S_HEAD_DIM) {
    const int d = threadIdx.x;
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < kSlots; ++i) s += red[i][d];
    const double m = s / static_cast<double>(valid_rows);
    const int64_t at = (static_cast<int64_t>(head) * blocks_total + global_block) * H3S_HEAD_DIM + d;
    switch (summary_dtype) {
      case H3S_F64: static_cast<double *>(summary)[at] = m; break;
      case H3S_F32: static_cast<float *>(summary)[at] = static_cast<float>(m); break;
      case H3S_BF16:
        static_cast<__nv_bfloat16 *>(summary)[at] = __float2bfloat16_rn(static_cast<float>(m));
        break;
      default:
        static_cast<__half *>(summary)[at] = __float2half_rn(static_cast<float>(m));
        break;
    }
  }
}

// ---------------------------------------------------------------------------
// FP8-E4M3 V carrier, transposed to (heads, 128, pad128(S)).
// One CTA = 128 sequence rows of one head, staged through shared memory so
// that both the row-major reads and the channel-major writes are full lines.
// ---------------------------------------------------------------------------

constexpr int kVTile = 128;
constexpr int kVThreads = 256;

// Shared tile: 128 channel rows of 128 bytes; the 16-byte chunk index of
// channel row d is XORed with (d>>3)&7 so the transposing 4-byte stores of
// the 16 lanes that share a sequence position fall in different banks.
__device__ __forceinline__ int v_tile_offset(int d, int s) {
  const int chunk = (s >> 4) ^ ((d >> 3) & 7);
  return d * kVTile + chunk * 16 + (s & 15);
}

template <typename T>
__global__ void __launch_bounds__(kVThreads)
quant_v_fp8_kernel(const T *__restrict__ v, int64_t stride_h, int64_t stride_s,
                   const float *__restrict__ v_scale, uint8_t *__restrict__ out, int rows,
                   int row_start, int padded_total, float v_bound) {
  __shared__ __align__(16) uint8_t tile[H3S_HEAD_DIM * kVTile];
  const int head = blockIdx.y;
  const int first_row = blockIdx.x * kVTile;
  const int valid_rows = max(0, min(kVTile, rows - first_row));
  const int slot = threadIdx.x >> 4;
  const int c0 = (threadIdx.x & 15) * 8;

  float sc[8], rc[8];
  bool all_exact = true;
  const bool clamp = v_bound < 448.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    sc[i] = fmaxf(__ldg(v_scale + head * H3S_HEAD_DIM + c0 + i), 1.0e-20f);
    const SharedDivisor d = make_divisor(sc[i]);
    rc[i] = d.r;
    all_exact = all_exact && d.exact;
  }

  const T *base = v + head * stride_h + c0;
  // the divisors' exactness is tested once, around the whole loop (see divide<>)
  auto fill = [&](auto exact_tag) {
  constexpr bool kExact = decltype(exact_tag)::value;
#pragma unroll
  for (int p = 0; p < kVTile / (kVThreads / 16 * 4); ++p) {
    const int r0 = (p * (kVThreads / 16) + slot) * 4;  // four consecutive rows
    // four consecutive rows of 8 channels -> per channel one word of four codes
    // (two 2-wide conversions and one byte permute)
    float q[4][8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (r0 + j < valid_rows) {
        float raw[8];
        Elem<T>::load8(base + static_cast<int64_t>(first_row + r0 + j) * stride_s, raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (kExact) {  // shared-divisor division, see SharedDivisor
            const float q0 = __fmul_rn(raw[i], rc[i]);
            q[j][i] = __fmaf_rn(__fmaf_rn(-sc[i], q0, raw[i]), rc[i], q0);
          } else {
            q[j][i] = __fdiv_rn(raw[i], sc[i]);
          }
          // the conversion saturates at +-448 by itself; a tighter bound is applied here
          if (clamp) q[j][i] = fminf(fmaxf(q[j][i], -v_bound), v_bound);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) q[j][i] = 0.f;
      }
    }
    uint32_t word[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint16_t lo, hi;
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(q[1][i]), "f"(q[0][i]));
      asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(q[3][i]), "f"(q[2][i]));
      word[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      *reinterpret_cast<uint32_t *>(&tile[v_tile_offset(c0 + i, r0)]) = word[i];
  }
  };
  if (all_exact) fill(std::true_type{}); else fill(std::false_type{});
  __syncthreads();
  uint8_t *dst = out + static_cast<int64_t>(head) * H3S_HEAD_DIM * padded_total + row_start + first_row;
#pragma unroll
  for (int p = 0; p < H3S_HEAD_DIM / (kVThreads / 8); ++p) {
    const int d = p * (kVThreads / 8) + (threadIdx.x >> 3);
    const int chunk = threadIdx.x & 7;
    const uint4 data = *reinterpret_cast<const uint4 *>(&tile[v_tile_offset(d, chunk * 16)]);
    *reinterpret_cast<uint4 *>(dst + static_cast<int64_t>(d) * padded_total + chunk * 16) = data;
  }
}

// ---------------------------------------------------------------------------
// Per-row FP8-E4M3 quantisation of a bf16 matrix (activations of the FP8 MLP).
// One CTA = one row, kept in registers between the amax reduction and the store.
// ---------------------------------------------------------------------------

constexpr int kRowQuantThreads = 256;
constexpr int kRowQuantMaxChunks = 8;  // 16-byte loads per thread: rows of up to 16384 channels

__global__ void __launch_bounds__(kRowQuantThreads)
quant_rows_fp8_kernel(const __nv_bfloat16 *__restrict__ x, int64_t stride_row, int rows, int channels,
                      uint8_t *__restrict__ out, float *__restrict__ row_scale) {
  __shared__ float warp_amax[kRowQuantThreads / 32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16 *src = x + row * stride_row;
    Elem<__nv_bfloat16>::Raw raw[kRowQuantMaxChunks];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < kRowQuantMaxChunks; ++i) {
      const int c0 = (i * kRowQuantThreads + threadIdx.x) * 8;
      raw[i] = c0 < channels ? Elem<__nv_bfloat16>::load_raw(src + c0) : Elem<__nv_bfloat16>::zero_raw();
      float v[8];
      Elem<__nv_bfloat16>::unpack(raw[i], v);
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
    }
    amax = warp_max(amax);
    __syncthreads();  // the previous row's readers are done
    if ((threadIdx.x & 31) == 0) warp_amax[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = warp_amax[0];
#pragma unroll
    for (int w = 1; w < kRowQuantThreads / 32; ++w) amax = fmaxf(amax, warp_amax[w]);
    const float scale = fmaxf(__fdiv_rn(amax, 448.0f), 1.0e-20f);
    if (threadIdx.x == 0) row_scale[row] = scale;
    const SharedDivisor by_scale = make_divisor(scale);
    auto emit = [&](auto exact_tag) {
      constexpr bool kExact = decltype(exact_tag)::value;
#pragma unroll
      for (int i = 0; i < kRowQuantMaxChunks; ++i) {
        const int c0 = (i * kRowQuantThreads + threadIdx.x) * 8;
        if (c0 < channels) {
          float v[8];
          Elem<__nv_bfloat16>::unpack(raw[i], v);
          uint32_t word[2];
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            uint16_t lo, hi;
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo)
                : "f"(divide<kExact>(by_scale, v[4 * w + 1])), "f"(divide<kExact>(by_scale, v[4 * w])));
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi)
                : "f"(divide<kExact>(by_scale, v[4 * w + 3])), "f"(divide<kExact>(by_scale, v[4 * w + 2])));
            word[w] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
          }
          *reinterpret_cast<uint2 *>(out + static_cast<int64_t>(row) * channels + c0) = make_uint2(word[0], word[1]);
        }
      }
    };
    if (by_scale.exact) emit(std::true_type{}); else emit(std::false_type{});
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

static int check_view(const void *p, int dtype, int64_t stride_h, int64_t stride_s, const char *what) {
  const int vec = dtype == H3S_F32 ? 4 : 8;  // elements per 16 bytes
  H3S_CHECK_ARG(dtype == H3S_F32 || dtype == H3S_BF16 || dtype == H3S_F16,
                "%s: unsupported dtype %d", what, dtype);
  H3S_CHECK_ARG((reinterpret_cast<uintptr_t>(p) & 15) == 0, "%s: pointer must be 16-byte aligned", what);
  H3S_CHECK_ARG(stride_h % vec == 0 && stride_s % vec == 0 && stride_s >= H3S_HEAD_DIM,
                "%s: strides (%lld,%lld) must be multiples of %d elements with row stride >= 128",
                what, static_cast<long long>(stride_h), static_cast<long long>(stride_s), vec);
  return H3S_OK;
}

template <typename T>
static int launch_column_stats(const void *k, int64_t ksh, int64_t kss, const void *v, int64_t vsh,
                               int64_t vss, int heads, int sequence, float v_bound, float *k_mean,
                               float *v_scale, void *scratch, cudaStream_t stream) {
  double *k_sum = static_cast<double *>(scratch);
  unsigned int *v_bits = reinterpret_cast<unsigned int *>(k_sum + heads * H3S_HEAD_DIM);
  H3S_CHECK_CUDA(cudaMemsetAsync(scratch, 0, h3s_column_stats_scratch_bytes(heads), stream));
  dim3 grid(ceil_div(sequence, kStatsRowsPerBlock), heads, 2);
  column_stats_kernel<T><<<grid, kStatsThreads, 0, stream>>>(
      static_cast<const T *>(k), ksh, kss, static_cast<const T *>(v), vsh, vss, sequence, k_sum, v_bits);
  const int total = heads * H3S_HEAD_DIM;
  column_stats_finalize_kernel<T><<<ceil_div(total, 256), 256, 0, stream>>>(
      k_sum, v_bits, total, sequence, v_bound, k == nullptr ? nullptr : k_mean,
      v == nullptr ? nullptr : v_scale);
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

template <typename T>
static int launch_quant_qk(const void *x, int64_t sh, int64_t ss, const float *mean, int8_t *out,
                           float *scale, void *summary, int summary_dtype, int heads, int rows,
                           int row_start, int sequence_total, int block, cudaStream_t stream) {
  const int blocks = ceil_div(rows, block);
  const int blocks_total = ceil_div(sequence_total, block);
  dim3 grid(blocks, heads);
#define H3S_LAUNCH_QK(BLOCK, HAS_MEAN)                                                               \
  quant_qk_blocks_kernel<T, BLOCK, HAS_MEAN><<<grid, BLOCK * 2, 0, stream>>>(                         \
      static_cast<const T *>(x), sh, ss, mean, out, scale, summary, summary_dtype, rows, row_start, \
      sequence_total, blocks_total)
  if (block == H3S_Q_TILE) {
    if (mean != nullptr) H3S_LAUNCH_QK(H3S_Q_TILE, true); else H3S_LAUNCH_QK(H3S_Q_TILE, false);
  } else {
    if (mean != nullptr) H3S_LAUNCH_QK(H3S_KV_TILE, true); else H3S_LAUNCH_QK(H3S_KV_TILE, false);
  }
#undef H3S_LAUNCH_QK
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

template <typename T>
static int launch_quant_v(const void *v, int64_t sh, int64_t ss, const float *v_scale, uint8_t *out,
                          int heads, int rows, int row_start, int sequence_total, float v_bound,
                          cudaStream_t stream) {
  const int padded_total = ceil_div(sequence_total, 128) * 128;
  // the final chunk also writes the zero padding up to the carrier's end
  const bool last = row_start + rows == sequence_total;
  const int covered = last ? padded_total - row_start : rows;
  dim3 grid(ceil_div(covered, kVTile), heads);
  quant_v_fp8_kernel<T><<<grid, kVThreads, 0, stream>>>(static_cast<const T *>(v), sh, ss, v_scale, out,
                                                        rows, row_start, padded_total, v_bound);
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

// ---------------------------------------------------------------------------
// Scratch that lives inside the library image, for hosts that cannot hand
// h3s_column_stats a scratch buffer of their own (see h3s_column_stats_static).
// Every device that loads this library carries one copy (96 KiB) until the
// process exits.  In host code the name below is only a stand-in for the
// symbol; the device address comes from cudaGetSymbolAddress, once per device.
// ---------------------------------------------------------------------------

constexpr int kStaticStatsMaxHeads = 64;
constexpr size_t kStaticStatsBytes =
    static_cast<size_t>(kStaticStatsMaxHeads) * H3S_HEAD_DIM * (sizeof(double) + sizeof(unsigned int));
static __device__ __align__(256) unsigned char g_static_stats_scratch[kStaticStatsBytes];

constexpr int kStaticStatsMaxDevices = 64;
static void *g_static_stats_addr[kStaticStatsMaxDevices] = {nullptr};
static std::mutex g_static_stats_mutex;

// Device address of the built-in scratch on the CURRENT device (looked up on
// the first call for that device, cached afterwards).
static int static_stats_scratch(void **out) {
  int device = 0;
  H3S_CHECK_CUDA(cudaGetDevice(&device));
  H3S_CHECK_ARG(device >= 0 && device < kStaticStatsMaxDevices,
                "column_stats_static: device ordinal %d is beyond the %d this library tracks", device,
                kStaticStatsMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_stats_mutex);
  if (g_static_stats_addr[device] == nullptr) {
    void *ptr = nullptr;
    H3S_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_static_stats_scratch));
    H3S_CHECK_ARG(ptr != nullptr, "column_stats_static: the built-in scratch has no device address");
    g_static_stats_addr[device] = ptr;
  }
  *out = g_static_stats_addr[device];
  return H3S_OK;
}

}  // namespace h3s

extern "C" {

size_t h3s_column_stats_scratch_bytes(int heads) {
  return static_cast<size_t>(heads) * H3S_HEAD_DIM * (sizeof(double) + sizeof(unsigned int));
}

int h3s_column_stats(const void *k, int64_t k_stride_h, int64_t k_stride_s, const void *v,
                     int64_t v_stride_h, int64_t v_stride_s, int dtype, int heads, int sequence,
                     float v_bound, float *k_mean, float *v_scale, void *scratch,
                     h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(heads > 0 && sequence > 0, "column_stats: empty problem (heads=%d sequence=%d)", heads, sequence);
  H3S_CHECK_ARG(k != nullptr || v != nullptr, "column_stats: both inputs are NULL");
  H3S_CHECK_ARG(scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 7) == 0,
                "column_stats: scratch must be non-NULL and 8-byte aligned");
  H3S_CHECK_ARG(k == nullptr || k_mean != nullptr, "column_stats: k given without k_mean");
  H3S_CHECK_ARG(v == nullptr || (v_scale != nullptr && v_bound > 0.f), "column_stats: v given without v_scale/bound");
  if (k != nullptr) { int rc = check_view(k, dtype, k_stride_h, k_stride_s, "column_stats k"); if (rc) return rc; }
  if (v != nullptr) { int rc = check_view(v, dtype, v_stride_h, v_stride_s, "column_stats v"); if (rc) return rc; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case H3S_F32: return launch_column_stats<float>(k, k_stride_h, k_stride_s, v, v_stride_h, v_stride_s, heads, sequence, v_bound, k_mean, v_scale, scratch, s);
    case H3S_BF16: return launch_column_stats<__nv_bfloat16>(k, k_stride_h, k_stride_s, v, v_stride_h, v_stride_s, heads, sequence, v_bound, k_mean, v_scale, scratch, s);
    default: return launch_column_stats<__half>(k, k_stride_h, k_stride_s, v, v_stride_h, v_stride_s, heads, sequence, v_bound, k_mean, v_scale, scratch, s);
  }
}

int h3s_quant_rows_fp8(const void *x_bf16, int64_t x_stride_row, int rows, int channels, uint8_t *out,
                       float *row_scale, h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(x_bf16 != nullptr && out != nullptr && row_scale != nullptr, "quant_rows_fp8: NULL pointer");
  H3S_CHECK_ARG(rows > 0 && channels > 0 && channels % 8 == 0 && channels <= kRowQuantThreads * 8 * kRowQuantMaxChunks,
                "quant_rows_fp8: channels %d must be a multiple of 8 and at most %d", channels,
                kRowQuantThreads * 8 * kRowQuantMaxChunks);
  H3S_CHECK_ARG((reinterpret_cast<uintptr_t>(x_bf16) & 15) == 0 && x_stride_row % 8 == 0 && x_stride_row >= channels,
                "quant_rows_fp8: input must be 16-byte aligned with a row stride that is a multiple of 8");
  H3S_CHECK_ARG((reinterpret_cast<uintptr_t>(out) & 7) == 0, "quant_rows_fp8: output must be 8-byte aligned");
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  quant_rows_fp8_kernel<<<grid, kRowQuantThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16 *>(x_bf16), x_stride_row, rows, channels, out, row_scale);
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

int h3s_column_stats_finalize(const void *stats, int dtype, int heads, int sequence, float v_bound,
                              float *k_mean, float *v_scale, h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(stats != nullptr && (reinterpret_cast<uintptr_t>(stats) & 7) == 0, "column_stats_finalize: stats must be non-NULL and 8-byte aligned");
  H3S_CHECK_ARG(heads > 0 && sequence > 0, "column_stats_finalize: empty problem");
  H3S_CHECK_ARG(k_mean != nullptr || v_scale != nullptr, "column_stats_finalize: nothing to produce");
  H3S_CHECK_ARG(v_scale == nullptr || v_bound > 0.f, "column_stats_finalize: v_bound must be positive");
  H3S_CHECK_ARG(dtype == H3S_F32 || dtype == H3S_BF16 || dtype == H3S_F16, "column_stats_finalize: unsupported dtype %d", dtype);
  const double *k_sum = static_cast<const double *>(stats);
  const unsigned int *v_bits = reinterpret_cast<const unsigned int *>(k_sum + heads * H3S_HEAD_DIM);
  const int total = heads * H3S_HEAD_DIM;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case H3S_F32: column_stats_finalize_kernel<float><<<ceil_div(total, 256), 256, 0, s>>>(k_sum, v_bits, total, sequence, v_bound, k_mean, v_scale); break;
    case H3S_BF16: column_stats_finalize_kernel<__nv_bfloat16><<<ceil_div(total, 256), 256, 0, s>>>(k_sum, v_bits, total, sequence, v_bound, k_mean, v_scale); break;
    default: column_stats_finalize_kernel<__half><<<ceil_div(total, 256), 256, 0, s>>>(k_sum, v_bits, total, sequence, v_bound, k_mean, v_scale); break;
  }
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

int h3s_quant_qk_blocks(const void *x, int dtype, int64_t x_stride_h, int64_t x_stride_s,
                        const float *mean, int8_t *out, float *scale, void *summary,
                        int summary_dtype, int heads, int rows, int row_start, int sequence_total,
                        int block, h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(block == H3S_Q_TILE || block == H3S_KV_TILE, "quant_qk_blocks: block must be 128 or 64, got %d", block);
  H3S_CHECK_ARG(heads > 0 && rows > 0 && sequence_total > 0, "quant_qk_blocks: empty problem");
  H3S_CHECK_ARG(row_start >= 0 && row_start % block == 0, "quant_qk_blocks: row_start %d is not a multiple of the block %d", row_start, block);
  H3S_CHECK_ARG(row_start + rows <= sequence_total, "quant_qk_blocks: chunk [%d,%d) exceeds sequence %d", row_start, row_start + rows, sequence_total);
  H3S_CHECK_ARG(rows % block == 0 || row_start + rows == sequence_total,
                "quant_qk_blocks: only the final chunk may contain a partial tile");
  H3S_CHECK_ARG(x != nullptr, "quant_qk_blocks: NULL input");
  H3S_CHECK_ARG((out != nullptr) == (scale != nullptr), "quant_qk_blocks: out and scale must be given together");
  H3S_CHECK_ARG(out != nullptr || summary != nullptr, "quant_qk_blocks: nothing to produce");
  H3S_CHECK_ARG((reinterpret_cast<uintptr_t>(out) & 7) == 0, "quant_qk_blocks: out must be 8-byte aligned");
  H3S_CHECK_ARG(summary == nullptr || (summary_dtype >= H3S_F32 && summary_dtype <= H3S_F64),
                "quant_qk_blocks: bad summary dtype %d", summary_dtype);
  { int rc = check_view(x, dtype, x_stride_h, x_stride_s, "quant_qk_blocks x"); if (rc) return rc; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case H3S_F32: return launch_quant_qk<float>(x, x_stride_h, x_stride_s, mean, out, scale, summary, summary_dtype, heads, rows, row_start, sequence_total, block, s);
    case H3S_BF16: return launch_quant_qk<__nv_bfloat16>(x, x_stride_h, x_stride_s, mean, out, scale, summary, summary_dtype, heads, rows, row_start, sequence_total, block, s);
    default: return launch_quant_qk<__half>(x, x_stride_h, x_stride_s, mean, out, scale, summary, summary_dtype, heads, rows, row_start, sequence_total, block, s);
  }
}

int h3s_quant_v_fp8(const void *v, int dtype, int64_t v_stride_h, int64_t v_stride_s,
                    const float *v_scale, uint8_t *out, int heads, int rows, int row_start,
                    int sequence_total, float v_bound, h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(heads > 0 && rows > 0 && sequence_total > 0, "quant_v_fp8: empty problem");
  H3S_CHECK_ARG(row_start >= 0 && row_start % 128 == 0, "quant_v_fp8: row_start %d must be 128 aligned", row_start);
  H3S_CHECK_ARG(row_start + rows <= sequence_total, "quant_v_fp8: chunk exceeds sequence");
  H3S_CHECK_ARG(rows % 128 == 0 || row_start + rows == sequence_total,
                "quant_v_fp8: only the final chunk may contain a partial tile");
  H3S_CHECK_ARG(v != nullptr && v_scale != nullptr && out != nullptr, "quant_v_fp8: NULL pointer");
  H3S_CHECK_ARG((reinterpret_cast<uintptr_t>(out) & 15) == 0, "quant_v_fp8: out must be 16-byte aligned");
  H3S_CHECK_ARG(v_bound > 0.f, "quant_v_fp8: v_bound must be positive");
  { int rc = check_view(v, dtype, v_stride_h, v_stride_s, "quant_v_fp8 v"); if (rc) return rc; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case H3S_F32: return launch_quant_v<float>(v, v_stride_h, v_stride_s, v_scale, out, heads, rows, row_start, sequence_total, v_bound, s);
    case H3S_BF16: return launch_quant_v<__nv_bfloat16>(v, v_stride_h, v_stride_s, v_scale, out, heads, rows, row_start, sequence_total, v_bound, s);
    default: return launch_quant_v<__half>(v, v_stride_h, v_stride_s, v_scale, out, heads, rows, row_start, sequence_total, v_bound, s);
  }
}


int h3s_column_stats_static(const void *k, int64_t k_stride_h, int64_t k_stride_s, const void *v,
                            int64_t v_stride_h, int64_t v_stride_s, int dtype, int heads, int sequence,
                            float v_bound, float *k_mean, float *v_scale, h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(heads > 0 && sequence > 0, "column_stats_static: empty problem (heads=%d sequence=%d)", heads, sequence);
  H3S_CHECK_ARG(heads <= kStaticStatsMaxHeads,
                "column_stats_static: %d heads exceed the %d the built-in scratch holds; use h3s_column_stats "
                "with a caller-provided scratch buffer instead", heads, kStaticStatsMaxHeads);
  H3S_CHECK_ARG(k != nullptr || v != nullptr, "column_stats_static: both inputs are NULL");
  H3S_CHECK_ARG(k == nullptr || k_mean != nullptr, "column_stats_static: k given without k_mean");
  H3S_CHECK_ARG(v == nullptr || (v_scale != nullptr && v_bound > 0.f), "column_stats_static: v given without v_scale/bound");
  if (k != nullptr) { int rc = check_view(k, dtype, k_stride_h, k_stride_s, "column_stats_static k"); if (rc) return rc; }
  if (v != nullptr) { int rc = check_view(v, dtype, v_stride_h, v_stride_s, "column_stats_static v"); if (rc) return rc; }
  void *scratch = nullptr;
  { int rc = static_stats_scratch(&scratch); if (rc) return rc; }
  // launch_column_stats clears the part of the scratch it uses (a memset on the
  // stream, not an allocation) before the accumulating kernel runs
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case H3S_F32: return launch_column_stats<float>(k, k_stride_h, k_stride_s, v, v_stride_h, v_stride_s, heads, sequence, v_bound, k_mean, v_scale, scratch, s);
    case H3S_BF16: return launch_column_stats<__nv_bfloat16>(k, k_stride_h, k_stride_s, v, v_stride_h, v_stride_s, heads, sequence, v_bound, k_mean, v_scale, scratch, s);
    default: return launch_column_stats<__half>(k, k_stride_h, k_stride_s, v, v_stride_h, v_stride_s, heads, sequence, v_bound, k_mean, v_scale, scratch, s);
  }
}

}  // extern "C"
