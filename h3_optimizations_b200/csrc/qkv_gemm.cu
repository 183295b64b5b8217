// Chunked ConvRot INT8 QKV projection for sm_100a.
//
//   convrot_quant_rows : x (rows, hidden) bf16 -> Hadamard-256 on every
//                        256-channel group (fast Walsh-Hadamard in registers
//                        and warp shuffles), per-row INT8 (scale = amax/127).
//                        HBM-bound, one warp per 256-channel group.
//   qkv_gemm_chunk     : persistent warp-specialised tcgen05 GEMM
//                        acc[rows, n] = x_i8 . w_i8^T (kind::i8, int32 in TMEM),
//                        128x256 tiles, K step 128 bytes (SWIZZLE_128B), 4-stage
//                        TMA ring, two TMEM accumulators so the epilogue of one
//                        tile overlaps the MMAs of the next.  The epilogue
//                        de-quantises (acc * (x_scale[row] * w_scale[col])), rounds
//                        to bf16 and scatters into head-major (3*H, rows, 128)
//                        staging that the carrier kernels consume.
//   qkv_gemm_chunk_carriers : the same GEMM whose epilogue emits the carriers
//                        themselves: INT8 Q blocks with scale and tile mean
//                        (a 128-row Q block of one head is one accumulator
//                        tile half), INT8 K half-blocks when K is not smoothed;
//                        K (when smoothed) and V, which need whole-sequence
//                        statistics, are staged as bf16 while their column sums
//                        / maxima are accumulated for the short second phase.
#include <cstring>

#include "common.cuh"
#include "ptx.cuh"
#include "tma.cuh"

namespace h3s {

// ---------------------------------------------------------------------------
// ConvRot prologue
// ---------------------------------------------------------------------------

constexpr int kRotGroup = 256;

// In-register part of the transform: butterflies over the three low index bits.
__device__ __forceinline__ void fwht8(float (&v)[8]) {
#pragma unroll
  for (int stride = 1; stride < 8; stride <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & stride) == 0) {
        const float a = v[i], b = v[i + stride];
        v[i] = __fadd_rn(a, b);
        v[i + stride] = __fsub_rn(a, b);
      }
    }
  }
}

__global__ void __launch_bounds__(384)
convrot_quant_rows_kernel(const __nv_bfloat16 *__restrict__ x, int64_t x_stride, int rows, int hidden,
                          int8_t *__restrict__ out, float *__restrict__ scale_out) {
  extern __shared__ float warp_amax[];  // one per warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = hidden / kRotGroup;  // == warps per CTA
  // the next row's 16 bytes are requested before this row is transformed, so every
  // thread keeps two loads in flight across the row's two barriers
  const __nv_bfloat16 *column = x + warp * kRotGroup + lane * 8;
  Elem<__nv_bfloat16>::Raw ahead = blockIdx.x < rows ? Elem<__nv_bfloat16>::load_raw(column + blockIdx.x * x_stride)
                                                     : Elem<__nv_bfloat16>::zero_raw();
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    float v[8];
    Elem<__nv_bfloat16>::unpack(ahead, v);
    const int next = row + gridDim.x;
    if (next < rows) ahead = Elem<__nv_bfloat16>::load_raw(column + static_cast<int64_t>(next) * x_stride);
    fwht8(v);
#pragma unroll
    for (int bit = 0; bit < 5; ++bit) {
      const bool upper = (lane >> bit) & 1;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, v[i], 1 << bit);
        v[i] = upper ? __fsub_rn(other, v[i]) : __fadd_rn(v[i], other);
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] *= 0.0625f;  // 1/sqrt(256), exact
      amax = fmaxf(amax, fabsf(v[i]));
    }
    amax = warp_max(amax);
    __syncthreads();  // previous row's readers are done
    if (lane == 0) warp_amax[warp] = amax;
    __syncthreads();
    amax = warp_amax[0];
    for (int w = 1; w < groups; ++w) amax = fmaxf(amax, warp_amax[w]);
    const float scale = amax > 0.f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const SharedDivisor by_scale = make_divisor(scale);  // exact v/scale without a divide per element
    uint32_t packed[2] = {0u, 0u};
    if (by_scale.exact) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        int code = __float2int_rn(divide<true>(by_scale, v[i]));
        code = max(-127, min(127, code));
        packed[i >> 2] |= (static_cast<uint32_t>(code) & 0xffu) << ((i & 3) * 8);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        int code = __float2int_rn(divide<false>(by_scale, v[i]));
        code = max(-127, min(127, code));
        packed[i >> 2] |= (static_cast<uint32_t>(code) & 0xffu) << ((i & 3) * 8);
      }
    }
    *reinterpret_cast<uint2 *>(out + static_cast<int64_t>(row) * hidden + warp * kRotGroup + lane * 8) =
        make_uint2(packed[0], packed[1]);
    if (threadIdx.x == 0) scale_out[row] = scale;
  }
}

// ---------------------------------------------------------------------------
// INT8 GEMM
// ---------------------------------------------------------------------------

constexpr int kGemmM = 128, kGemmN = 256, kGemmK = 128;  // K in bytes == int8 elements
// warps 0-3: epilogue of the tile's first 128 columns, 4: TMA, 5: MMA, 6-7: idle,
// 8-11: epilogue of the second 128 columns (a warp may only touch the TMEM lanes
// 32*(warp%4)..: two warps per lane quarter halve the epilogue's time, which
// exceeds the MMA time of a tile once the norm and the rotation run in it)
constexpr int kGemmThreads = 384;
constexpr uint32_t kGemmABytes = kGemmM * kGemmK;  // 16384
constexpr uint32_t kGemmBBytes = kGemmN * kGemmK;  // 32768
constexpr uint32_t kGemmTmemCols = 512;

// What the eight 16-thread row slots of one 128-column half of a tile tell each
// other in the carrier epilogue: per-warp largest magnitudes and per-slot
// per-channel partial sums (maxima for V) of the rows 0-63 and 64-127 of the tile.
struct EpilogueExchange {
  float amax[2][4];                 // [row half][warp]
  float column[2][8][H3S_HEAD_DIM];  // [row half][slot][channel]
};
constexpr uint32_t kEpilogueTileBytes = kGemmM * H3S_HEAD_DIM * 2;  // one half tile as bf16: 32 KB

// Shared-memory layout.  The carrier epilogue stages each half tile as bf16 so
// that it can be re-read column-wise (quantisation, statistics and every global
// store then run on contiguous lines); it pays for the two 32 KB staging tiles
// with one stage of the operand ring.
// Epilogue of the GEMM kernel
enum GemmMode {
  kModeStaging = 0,   // INT8 x INT8 -> bf16 head-major staging (h3s_qkv_gemm_chunk[_norm_rope])
  kModeCarriers = 1,  // INT8 x INT8 -> carriers (h3s_qkv_gemm_chunk_carriers)
  kModeDense = 2,     // any operand kind -> scaled, biased, activated bf16 row-major matrix (h3s_dense_gemm)
};

template <int kMode>
struct GemmLayout {
  static constexpr bool kCarriers = kMode != kModeStaging;  // both stage half tiles for coalesced stores
  static constexpr int kStages = kCarriers ? 3 : 4;
  static constexpr uint32_t kOffB = kStages * kGemmABytes;
  static constexpr uint32_t kOffTile = kOffB + kStages * kGemmBBytes;
  static constexpr uint32_t kOffExchange = kOffTile + (kCarriers ? 2 * kEpilogueTileBytes : 0);
  static constexpr uint32_t kOffBar = kOffExchange + (kCarriers ? 2 * sizeof(EpilogueExchange) : 0);
  static constexpr uint32_t kBytes = kOffBar + 256 + 1024;
  static_assert(kBytes <= 227 * 1024, "GEMM shared memory exceeds the per-CTA limit");
};
constexpr int kGemmMaxStages = 4;

enum GemmAbort { kGemmAbortFull = 21, kGemmAbortEmpty, kGemmAbortAccFull, kGemmAbortAccEmpty, kGemmAbortTile, kGemmAbortExchange };

struct GemmShared {
  uint64_t full[kGemmMaxStages];
  uint64_t empty[kGemmMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t tile_ready[2];      // per tile half: its four warps have staged their rows
  uint64_t exchange_ready[2];  // per tile half: its four warps have written their EpilogueExchange
  uint32_t tmem_base;
  int abort_word;
};

struct GemmParams {
  const float *x_scale;   // (rows)
  const float *w_scale;   // (n_out)
  __nv_bfloat16 *out;     // (n_out/128, out_rows_stride/128.., 128): head-major staging
  int64_t out_stride_head;  // elements between consecutive 128-column groups
  int32_t *status;
  int rows, n_out, hidden;
  int m_tiles, n_tiles;
  // Column tiles are visited in the order (i * n_step) % n_tiles (n_step coprime with
  // n_tiles, about a third of it): weight rows are ordered [Q | K | V], so consecutive
  // tiles of a CTA alternate between the three kinds and the costlier epilogues of
  // one kind spread out instead of arriving in a row.
  int n_step;
  // optional per-head RMS norm (+ split-half rotation) of the Q and K groups
  const float *q_norm;    // (128) or null: no norm, no rotation
  const float *k_norm;    // (128)
  const void *rope;       // (rows, 48, 2, 2) view with the strides below, or null
  int64_t rope_stride_seq, rope_stride_dim, rope_stride_rot, rope_stride_pair;
  int rope_dtype;         // H3S_F32 or H3S_BF16
  int heads;
  float epsilon;
  unsigned long long wait_budget_ns;  // bound of every mbarrier wait
  // carrier epilogue (h3s_qkv_gemm_chunk_carriers); all tensors cover the whole sequence
  int8_t *q8, *k8;                 // (heads, sequence_total, 128); k8 null: K is staged
  float *q_scale, *k_scale;        // (heads, ceil(S/128)), (heads, ceil(S/64))
  void *q_summary, *k_summary;     // (heads, blocks, 128) tile means, summary_dtype
  __nv_bfloat16 *k_stage, *v_stage;  // (heads, sequence_total, 128)
  double *k_sum;                   // (heads, 128) running column sums of K, or null
  unsigned int *v_amax_bits;       // (heads, 128) running column maxima of |V| as float bits
  int summary_dtype, sequence_total, row_start;
  // dense epilogue (h3s_dense_gemm): out[m, n] = act(acc * row_scale[m] * col_scale[n] + bias[n]) as bf16
  int operand_kind;                // H3S_GEMM_I8 / BF16 / F16 / E4M3
  const float *row_scale;          // (rows) or null
  const float *col_scale;          // (n_out) or null
  const float *bias;               // (n_out) or null
  int activation;                  // H3S_ACT_NONE / H3S_ACT_GELU_TANH
  __nv_bfloat16 *dense_out;        // (rows, ldc)
  int64_t ldc;
};

__device__ __forceinline__ float gelu_tanh(float x) {
  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), the formula of torch's approximate='tanh'
  const float inner = 0.7978845608028654f * __fmaf_rn(0.044715f * x, x * x, x);
  return 0.5f * x * (1.0f + tanhf(inner));
}

__device__ __forceinline__ float rope_load(const void *base, int64_t index, int dtype) {
  return dtype == H3S_F32 ? __ldg(static_cast<const float *>(base) + index)
                          : __bfloat162float(__ldg(static_cast<const __nv_bfloat16 *>(base) + index));
}

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&t);
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ void store_summary(void *base, int dtype, int64_t at, double value) {
  switch (dtype) {
    case H3S_F64: static_cast<double *>(base)[at] = value; break;
    case H3S_F32: static_cast<float *>(base)[at] = static_cast<float>(value); break;
    case H3S_BF16: static_cast<__nv_bfloat16 *>(base)[at] = __float2bfloat16_rn(static_cast<float>(value)); break;
    default: static_cast<__half *>(base)[at] = __float2half_rn(static_cast<float>(value)); break;
  }
}

// INT8 codes of eight consecutive channels held as four bf16 pairs:
// code = trunc(v/scale +- 0.5) with the correctly rounded quotient (the arithmetic
// of quant_qk_blocks_kernel), written as one 8-byte store.
template <bool kExact>
__device__ __forceinline__ void quantise8(const uint4 &raw, const SharedDivisor &by_scale, int8_t *dst) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t code[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float q = divide<kExact>(by_scale, (i & 1) ? bf16_hi(w[i >> 1]) : bf16_lo(w[i >> 1]));
    const float half_ulp = __uint_as_float((__float_as_uint(q) & 0x80000000u) | 0x3f000000u);  // +-0.5
    q = __fadd_rn(q, half_ulp);
    code[i] = static_cast<uint32_t>(static_cast<int>(q));  // truncation toward zero
  }
  uint32_t packed[2];
#pragma unroll
  for (int k = 0; k < 2; ++k)
    packed[k] = __byte_perm(__byte_perm(code[4 * k], code[4 * k + 1], 0x0040),
                            __byte_perm(code[4 * k + 2], code[4 * k + 3], 0x0040), 0x5410);
  *reinterpret_cast<uint2 *>(dst) = make_uint2(packed[0], packed[1]);
}

// One row of one Q or K head after the GEMM, held as 64 bf16 pairs (every
// intermediate of the reference epilogue is rounded to bf16, so the packed
// form loses nothing): RMS norm over the 128 channels with the per-channel
// weight, then the split-half rotation of channels [0,48) against [48,96).
// Same order of operations and roundings as the reference
// (attention/sparse/fused_qkv.py:218-289); the sum of squares is accumulated
// in FP64 so that it does not depend on the order of the additions.
__device__ __forceinline__ void norm_rope_row(uint32_t (&y)[H3S_HEAD_DIM / 2], const float *__restrict__ norm_weight,
                                              float epsilon, const void *rope_row, int rope_dtype,
                                              int64_t stride_dim, int64_t stride_rot, int64_t stride_pair) {
  double sum = 0.0;
#pragma unroll
  for (int i = 0; i < H3S_HEAD_DIM / 2; ++i) {
    const double lo = static_cast<double>(bf16_lo(y[i])), hi = static_cast<double>(bf16_hi(y[i]));
    sum = fma(lo, lo, sum);
    sum = fma(hi, hi, sum);
  }
  const float mean = __fadd_rn(__fmul_rn(static_cast<float>(sum), 1.0f / H3S_HEAD_DIM), epsilon);
  const float inverse_rms = __frsqrt_rn(mean);
#pragma unroll
  for (int i = 0; i < H3S_HEAD_DIM / 2; ++i) {
    const float2 w = __ldg(reinterpret_cast<const float2 *>(norm_weight) + i);
    y[i] = pack_bf16x2(__fmul_rn(__fmul_rn(bf16_lo(y[i]), inverse_rms), w.x),
                       __fmul_rn(__fmul_rn(bf16_hi(y[i]), inverse_rms), w.y));
  }
  if (rope_row != nullptr) {
    // (48,2,2) tables stored contiguously (the layout the model produces) are
    // read 16 bytes at a time: the eight factors of channels 2i and 2i+1
    const bool packed = stride_pair == 1 && stride_rot == 2 && stride_dim == 4 &&
                        (reinterpret_cast<uintptr_t>(rope_row) & 15) == 0;
#pragma unroll
    for (int i = 0; i < 24; ++i) {  // channels 2i, 2i+1 against 2i+48, 2i+49
      float f[2][4];  // [channel][f00, f01, f10, f11]
      if (packed && rope_dtype == H3S_BF16) {
        const uint4 w = __ldg(reinterpret_cast<const uint4 *>(rope_row) + i);
        f[0][0] = bf16_lo(w.x); f[0][1] = bf16_hi(w.x); f[0][2] = bf16_lo(w.y); f[0][3] = bf16_hi(w.y);
        f[1][0] = bf16_lo(w.z); f[1][1] = bf16_hi(w.z); f[1][2] = bf16_lo(w.w); f[1][3] = bf16_hi(w.w);
      } else if (packed) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(rope_row) + 2 * i);
        const float4 b = __ldg(reinterpret_cast<const float4 *>(rope_row) + 2 * i + 1);
        f[0][0] = a.x; f[0][1] = a.y; f[0][2] = a.z; f[0][3] = a.w;
        f[1][0] = b.x; f[1][1] = b.y; f[1][2] = b.z; f[1][3] = b.w;
      } else {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int64_t at = (2 * i + e) * stride_dim;
          f[e][0] = rope_load(rope_row, at, rope_dtype);
          f[e][1] = rope_load(rope_row, at + stride_pair, rope_dtype);
          f[e][2] = rope_load(rope_row, at + stride_rot, rope_dtype);
          f[e][3] = rope_load(rope_row, at + stride_rot + stride_pair, rope_dtype);
        }
      }
      const float first[2] = {bf16_lo(y[i]), bf16_hi(y[i])};
      const float second[2] = {bf16_lo(y[i + 24]), bf16_hi(y[i + 24])};
      float out_first[2], out_second[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        out_first[e] = __fadd_rn(__fmul_rn(f[e][0], first[e]), __fmul_rn(f[e][1], second[e]));
        out_second[e] = __fadd_rn(__fmul_rn(f[e][2], first[e]), __fmul_rn(f[e][3], second[e]));
      }
      y[i] = pack_bf16x2(out_first[0], out_first[1]);
      y[i + 24] = pack_bf16x2(out_second[0], out_second[1]);
    }
  }
}

template <int kMode>
__global__ void __launch_bounds__(kGemmThreads, 1)
qkv_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const GemmParams prm) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
  using L = GemmLayout<kMode>;
  constexpr bool kCarriers = kMode == kModeCarriers;
  GemmShared &sh = *reinterpret_cast<GemmShared *>(smem + L::kOffBar);
  volatile int *abort_word = &sh.abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_steps = prm.hidden / kGemmK;
  const int total_tiles = prm.m_tiles * prm.n_tiles;

  if (threadIdx.x == 0) {
    for (int i = 0; i < L::kStages; ++i) {
      ptx::mbar_init(&sh.full[i], 1);
      ptx::mbar_init(&sh.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&sh.acc_full[i], 1);
      ptx::mbar_init(&sh.acc_empty[i], 8);
      ptx::mbar_init(&sh.tile_ready[i], 4);
      ptx::mbar_init(&sh.exchange_ready[i], 4);
    }
    sh.abort_word = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 5) {
    ptx::tmem_alloc(&sh.tmem_base, kGemmTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (warp == 4) {
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_a);
      ptx::prefetch_tensormap(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int tm = tile % prm.m_tiles, tn = (tile / prm.m_tiles) * prm.n_step % prm.n_tiles;
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % L::kStages;
          const uint32_t use = it / L::kStages;
          if (!ptx::mbar_wait(&sh.empty[s], (use & 1u) ^ 1u, abort_word, kGemmAbortEmpty, prm.wait_budget_ns)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(&sh.full[s], kGemmABytes + kGemmBBytes);
          ptx::tma_load_2d(smem + s * kGemmABytes, &map_a, &sh.full[s], ks * kGemmK, tm * kGemmM);
          ptx::tma_load_2d(smem + L::kOffB + s * kGemmBBytes, &map_b, &sh.full[s], ks * kGemmK, tn * kGemmN);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // every kind consumes 32 bytes of K per instruction: four instructions per 128-byte stage
      const int kind = kMode == kModeDense ? prm.operand_kind : H3S_GEMM_I8;
      const uint32_t idesc = kind == H3S_GEMM_I8     ? ptx::umma_idesc(2, 1, 1, kGemmM, kGemmN)
                             : kind == H3S_GEMM_E4M3 ? ptx::umma_idesc(1, 0, 0, kGemmM, kGemmN)
                             : kind == H3S_GEMM_BF16 ? ptx::umma_idesc(1, 1, 1, kGemmM, kGemmN)
                                                     : ptx::umma_idesc(1, 0, 0, kGemmM, kGemmN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local) {
        const int a = local & 1;
        const uint32_t acc_use = local >> 1;
        if (!ptx::mbar_wait(&sh.acc_empty[a], (acc_use & 1u) ^ 1u, abort_word, kGemmAbortAccEmpty, prm.wait_budget_ns)) { ok = false; break; }
        ptx::tc_fence_after();
        for (int ks = 0; ks < k_steps; ++ks, ++it) {
          const int s = it % L::kStages;
          const uint32_t use = it / L::kStages;
          if (!ptx::mbar_wait(&sh.full[s], use & 1u, abort_word, kGemmAbortFull, prm.wait_budget_ns)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint64_t a_desc = ptx::umma_desc_kmajor(ptx::smem_u32(smem + s * kGemmABytes), 1024, ptx::kSwizzle128);
          const uint64_t b_desc =
              ptx::umma_desc_kmajor(ptx::smem_u32(smem + L::kOffB + s * kGemmBBytes), 1024, ptx::kSwizzle128);
          if (kind == H3S_GEMM_I8) {
#pragma unroll
            for (int k = 0; k < kGemmK / 32; ++k)
              ptx::umma_i8(tmem_base + a * kGemmN, a_desc + 2 * k, b_desc + 2 * k, idesc, (ks > 0 || k > 0) ? 1u : 0u);
          } else if (kind == H3S_GEMM_E4M3) {
#pragma unroll
            for (int k = 0; k < kGemmK / 32; ++k)
              ptx::umma_f8(tmem_base + a * kGemmN, a_desc + 2 * k, b_desc + 2 * k, idesc, (ks > 0 || k > 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int k = 0; k < kGemmK / 32; ++k)
              ptx::umma_f16(tmem_base + a * kGemmN, a_desc + 2 * k, b_desc + 2 * k, idesc, (ks > 0 || k > 0) ? 1u : 0u);
          }
          ptx::tc_commit(&sh.empty[s]);
        }
        if (ok) ptx::tc_commit(&sh.acc_full[a]);
      }
    }
  } else if (warp < 4 || warp >= 8) {
    // epilogue: thread <-> accumulator row, warp group <-> 128-column half of the tile
    const int quarter = warp & 3;
    const int gi = warp >= 8 ? 1 : 0;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t local = 0;
    uint32_t exchanges = 0;  // uses of this half's exchange buffer and barrier so far
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local) {
      const int tm = tile % prm.m_tiles, tn = (tile / prm.m_tiles) * prm.n_step % prm.n_tiles;
      const int a = local & 1;
      const uint32_t acc_use = local >> 1;
      {
        const bool got = ptx::mbar_wait(&sh.acc_full[a], acc_use & 1u, abort_word, kGemmAbortAccFull, prm.wait_budget_ns);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      }
      ptx::tc_fence_after();
      const int row = tm * kGemmM + quarter * 32 + lane;
      const bool row_ok = row < prm.rows;
      const float xs = prm.x_scale == nullptr ? 1.0f : (row_ok ? __ldg(prm.x_scale + row) : 0.f);
      {
        const int group_col0 = tn * kGemmN + gi * H3S_HEAD_DIM;
        const int group = group_col0 >> 7;  // 128-column group == (kind, head)
        const bool group_ok = group_col0 < prm.n_out;
        const bool normed = prm.q_norm != nullptr && group < 2 * prm.heads;
        if (kMode == kModeDense) {
          // ---- dense epilogue: scaled, biased, activated bf16 rows, staged for coalesced stores ----
          unsigned char *tile = smem + L::kOffTile + gi * kEpilogueTileBytes;
          const int local_row = quarter * 32 + lane;
          const float rs = xs;  // row_scale[row], 1 without row scales
          const bool integer = prm.operand_kind == H3S_GEMM_I8;
          uint4 *my_row = reinterpret_cast<uint4 *>(tile + local_row * (H3S_HEAD_DIM * 2));
#pragma unroll 1
          for (int cc = 0; cc < H3S_HEAD_DIM / 32; ++cc) {
            uint32_t acc[32];
            H3S_TMEM_LD32(tmem_base + lane_addr + a * kGemmN + gi * H3S_HEAD_DIM + cc * 32, acc);
            ptx::tmem_wait_ld();
            uint32_t y[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float v[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int col = group_col0 + cc * 32 + i + e;
                const bool col_ok = col < prm.n_out;
                float value = integer ? static_cast<float>(static_cast<int>(acc[i + e])) : __uint_as_float(acc[i + e]);
                const float cs = (prm.col_scale != nullptr && col_ok) ? __ldg(prm.col_scale + col) : 1.0f;
                value = __fmul_rn(value, __fmul_rn(rs, cs));
                if (prm.bias != nullptr && col_ok) value = __fadd_rn(value, __ldg(prm.bias + col));
                if (prm.activation == H3S_ACT_GELU_TANH) value = gelu_tanh(value);
                v[e] = value;
              }
              y[i >> 1] = pack_bf16x2(v[0], v[1]);
            }
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
              my_row[(cc * 4 + c4) ^ (local_row & 15)] = make_uint4(y[4 * c4], y[4 * c4 + 1], y[4 * c4 + 2], y[4 * c4 + 3]);
          }
          // the accumulator has been read: the MMA warp may refill it
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&sh.acc_empty[a]);
          if (!group_ok) continue;  // the same for the four warps of this half
          if (lane == 0) ptx::mbar_arrive(&sh.tile_ready[gi]);
          {
            const bool got = ptx::mbar_wait(&sh.tile_ready[gi], exchanges & 1u, abort_word, kGemmAbortTile,
                                            prm.wait_budget_ns);
            if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
          }
          // 16 threads per row, 16 bytes each: a warp writes two rows of 256 contiguous bytes
          const int g = quarter * 32 + lane, slot = g >> 4, c = g & 15;
          uint4 raw[16];
#pragma unroll
          for (int p = 0; p < 16; ++p) {
            const int r = p * 8 + slot;
            raw[p] = *reinterpret_cast<const uint4 *>(tile + r * (H3S_HEAD_DIM * 2) + ((c ^ (r & 15)) << 4));
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&sh.exchange_ready[gi]);
          {
            const bool got = ptx::mbar_wait(&sh.exchange_ready[gi], exchanges & 1u, abort_word, kGemmAbortExchange,
                                            prm.wait_budget_ns);
            if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
            ++exchanges;
          }
          const int valid = min(kGemmM, prm.rows - tm * kGemmM);
          const int col = group_col0 + c * 8;
          if (col < prm.n_out) {  // n_out is a multiple of 8: a 16-byte chunk is inside or outside as a whole
            __nv_bfloat16 *dst = prm.dense_out + static_cast<int64_t>(tm) * kGemmM * prm.ldc + col;
#pragma unroll
            for (int p = 0; p < 16; ++p) {
              const int r = p * 8 + slot;
              if (r < valid) *reinterpret_cast<uint4 *>(dst + static_cast<int64_t>(r) * prm.ldc) = raw[p];
            }
          }
          continue;  // acc_empty was signalled above
        }
        if (kCarriers) {
          // ---- carriers straight from the accumulators ----
          // Phase A, one thread per row: de-quantise the row of this head to bf16
          // (+ norm and rotation) and stage it in shared memory, 16-byte chunk c of
          // row r at chunk position c ^ (r & 15) so that neither these row-wise
          // writes nor the column-wise reads of phase B collide on banks.
          unsigned char *tile = smem + L::kOffTile + gi * kEpilogueTileBytes;
          const int local_row = quarter * 32 + lane;
          {
            uint32_t y[H3S_HEAD_DIM / 2];
#pragma unroll
            for (int cc = 0; cc < H3S_HEAD_DIM / 32; ++cc) {
              uint32_t acc[32];
              H3S_TMEM_LD32(tmem_base + lane_addr + a * kGemmN + gi * H3S_HEAD_DIM + cc * 32, acc);
              ptx::tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float2 ws = group_ok ? __ldg(reinterpret_cast<const float2 *>(prm.w_scale + group_col0 + cc * 32 + i))
                                           : make_float2(0.f, 0.f);
                y[cc * 16 + (i >> 1)] =
                    pack_bf16x2(__fmul_rn(static_cast<float>(static_cast<int>(acc[i])), __fmul_rn(xs, ws.x)),
                                __fmul_rn(static_cast<float>(static_cast<int>(acc[i + 1])), __fmul_rn(xs, ws.y)));
              }
            }
            // the accumulator is in registers: the MMA warp may refill it
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&sh.acc_empty[a]);
            if (!group_ok) continue;  // the same for the four warps of this half
            if (normed && row_ok) {
              const void *rope_row = nullptr;
              if (prm.rope != nullptr) {
                const int64_t offset = static_cast<int64_t>(row) * prm.rope_stride_seq;
                rope_row = prm.rope_dtype == H3S_F32
                               ? static_cast<const void *>(static_cast<const float *>(prm.rope) + offset)
                               : static_cast<const void *>(static_cast<const __nv_bfloat16 *>(prm.rope) + offset);
              }
              norm_rope_row(y, group < prm.heads ? prm.q_norm : prm.k_norm, prm.epsilon, rope_row, prm.rope_dtype,
                            prm.rope_stride_dim, prm.rope_stride_rot, prm.rope_stride_pair);
            }
            uint4 *my_row = reinterpret_cast<uint4 *>(tile + local_row * (H3S_HEAD_DIM * 2));
#pragma unroll
            for (int c = 0; c < 16; ++c)
              my_row[c ^ (local_row & 15)] = row_ok ? make_uint4(y[4 * c], y[4 * c + 1], y[4 * c + 2], y[4 * c + 3])
                                                    : make_uint4(0u, 0u, 0u, 0u);  // rows past the chunk count as zeros
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&sh.tile_ready[gi]);
          {
            const bool got = ptx::mbar_wait(&sh.tile_ready[gi], exchanges & 1u, abort_word, kGemmAbortTile,
                                            prm.wait_budget_ns);
            if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
          }
          // Phase B, 16 threads per row, 8 channels each: thread (slot, c) holds rows
          // slot, slot+8, ... slot+120 of channels 8c..8c+7, as in quant_qk_blocks_kernel.
          const int kind = group / prm.heads, head = group - kind * prm.heads;
          const int g = quarter * 32 + lane;  // thread within this half's 128
          const int slot = g >> 4, c = g & 15;
          const bool quantise_here = kind == 0 || (kind == 1 && prm.k8 != nullptr);
          EpilogueExchange &ex = reinterpret_cast<EpilogueExchange *>(smem + L::kOffExchange)[gi];
          uint4 raw[16];
#pragma unroll
          for (int p = 0; p < 16; ++p) {
            const int r = p * 8 + slot;
            raw[p] = *reinterpret_cast<const uint4 *>(tile + r * (H3S_HEAD_DIM * 2) + ((c ^ (r & 15)) << 4));
          }
          {
            // partial statistics of rows 0-63 (passes 0-7) and 64-127 (passes 8-15)
            float part[2][8];
            __nv_bfloat162 top[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              top[h] = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
              for (int i = 0; i < 8; ++i) part[h][i] = 0.f;
#pragma unroll
              for (int p = 8 * h; p < 8 * h + 8; ++p) {
                const uint32_t w[4] = {raw[p].x, raw[p].y, raw[p].z, raw[p].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  if (kind == 2) {
                    part[h][2 * i] = fmaxf(part[h][2 * i], fabsf(bf16_lo(w[i])));
                    part[h][2 * i + 1] = fmaxf(part[h][2 * i + 1], fabsf(bf16_hi(w[i])));
                  } else {
                    part[h][2 * i] = __fadd_rn(part[h][2 * i], bf16_lo(w[i]));
                    part[h][2 * i + 1] = __fadd_rn(part[h][2 * i + 1], bf16_hi(w[i]));
                    if (quantise_here) {  // magnitudes two at a time: clear both sign bits, packed bf16 maximum
                      const uint32_t magnitude = w[i] & 0x7fff7fffu;
                      top[h] = __hmax2(top[h], *reinterpret_cast<const __nv_bfloat162 *>(&magnitude));
                    }
                  }
                }
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) ex.column[h][slot][c * 8 + i] = part[h][i];
              if (quantise_here) {
                const uint32_t bits = *reinterpret_cast<const uint32_t *>(&top[h]);
                const float amax = warp_max(fmaxf(bf16_lo(bits), bf16_hi(bits)));
                if (lane == 0) ex.amax[h][quarter] = amax;
              }
            }
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&sh.exchange_ready[gi]);
          {
            const bool got = ptx::mbar_wait(&sh.exchange_ready[gi], exchanges & 1u, abort_word, kGemmAbortExchange,
                                            prm.wait_budget_ns);
            if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
            ++exchanges;
          }
          // every thread of this half now holds its share of the tile in registers: the
          // staging tile may be overwritten, the exchange block is read below
          const int tile_row0 = prm.row_start + tm * kGemmM;  // first row of this tile within the sequence
          const int valid = min(kGemmM, prm.rows - tm * kGemmM);
          const int valid_half[2] = {min(H3S_KV_TILE, valid), max(0, valid - H3S_KV_TILE)};
          float amax_half[2] = {0.f, 0.f};
          if (quantise_here) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
              amax_half[h] = fmaxf(fmaxf(ex.amax[h][0], ex.amax[h][1]), fmaxf(ex.amax[h][2], ex.amax[h][3]));
          }
          // channel g of this head: totals over the eight row slots
          double total[2] = {0.0, 0.0};
          float peak = 0.f;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) {
              if (kind == 2) peak = fmaxf(peak, ex.column[h][sl][g]);
              else total[h] += static_cast<double>(ex.column[h][sl][g]);
            }
          }
          if (kind == 0) {
            const int blocks_total = (prm.sequence_total + H3S_Q_TILE - 1) / H3S_Q_TILE;
            const int block = tile_row0 / H3S_Q_TILE;
            const float scale = __fadd_rn(__fdiv_rn(fmaxf(amax_half[0], amax_half[1]), 127.0f), 1.0e-7f);
            if (g == 0) prm.q_scale[head * blocks_total + block] = scale;
            store_summary(prm.q_summary, prm.summary_dtype,
                          (static_cast<int64_t>(head) * blocks_total + block) * H3S_HEAD_DIM + g, (total[0] + total[1]) / valid);
            int8_t *dst = prm.q8 + (static_cast<int64_t>(head) * prm.sequence_total + tile_row0) * H3S_HEAD_DIM + c * 8;
            const SharedDivisor by_scale = make_divisor(scale);
            if (by_scale.exact) {
#pragma unroll
              for (int p = 0; p < 16; ++p) {
                const int r = p * 8 + slot;
                if (r < valid) quantise8<true>(raw[p], by_scale, dst + static_cast<int64_t>(r) * H3S_HEAD_DIM);
              }
            } else {
#pragma unroll
              for (int p = 0; p < 16; ++p) {
                const int r = p * 8 + slot;
                if (r < valid) quantise8<false>(raw[p], by_scale, dst + static_cast<int64_t>(r) * H3S_HEAD_DIM);
              }
            }
          } else if (kind == 1) {
            const int blocks_total = (prm.sequence_total + H3S_KV_TILE - 1) / H3S_KV_TILE;
            const int block0 = tile_row0 / H3S_KV_TILE;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (valid_half[h] > 0)
                store_summary(prm.k_summary, prm.summary_dtype,
                              (static_cast<int64_t>(head) * blocks_total + block0 + h) * H3S_HEAD_DIM + g, total[h] / valid_half[h]);
            }
            if (prm.k_sum != nullptr) atomicAdd(prm.k_sum + head * H3S_HEAD_DIM + g, total[0] + total[1]);
            if (prm.k8 != nullptr) {
              int8_t *dst = prm.k8 + (static_cast<int64_t>(head) * prm.sequence_total + tile_row0) * H3S_HEAD_DIM + c * 8;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const float scale = __fadd_rn(__fdiv_rn(amax_half[h], 127.0f), 1.0e-7f);
                if (g == 0 && valid_half[h] > 0) prm.k_scale[head * blocks_total + block0 + h] = scale;
                const SharedDivisor by_scale = make_divisor(scale);
                if (by_scale.exact) {
#pragma unroll
                  for (int p = 8 * h; p < 8 * h + 8; ++p) {
                    const int r = p * 8 + slot;
                    if (r < valid) quantise8<true>(raw[p], by_scale, dst + static_cast<int64_t>(r) * H3S_HEAD_DIM);
                  }
                } else {
#pragma unroll
                  for (int p = 8 * h; p < 8 * h + 8; ++p) {
                    const int r = p * 8 + slot;
                    if (r < valid) quantise8<false>(raw[p], by_scale, dst + static_cast<int64_t>(r) * H3S_HEAD_DIM);
                  }
                }
              }
            } else {
              __nv_bfloat16 *dst = prm.k_stage + (static_cast<int64_t>(head) * prm.sequence_total + tile_row0) * H3S_HEAD_DIM + c * 8;
#pragma unroll
              for (int p = 0; p < 16; ++p) {
                const int r = p * 8 + slot;
                if (r < valid) *reinterpret_cast<uint4 *>(dst + static_cast<int64_t>(r) * H3S_HEAD_DIM) = raw[p];
              }
            }
          } else {
            // non-negative floats order like their bit patterns
            atomicMax(prm.v_amax_bits + head * H3S_HEAD_DIM + g, __float_as_uint(peak));
            __nv_bfloat16 *dst = prm.v_stage + (static_cast<int64_t>(head) * prm.sequence_total + tile_row0) * H3S_HEAD_DIM + c * 8;
#pragma unroll
            for (int p = 0; p < 16; ++p) {
              const int r = p * 8 + slot;
              if (r < valid) *reinterpret_cast<uint4 *>(dst + static_cast<int64_t>(r) * H3S_HEAD_DIM) = raw[p];
            }
          }
          continue;  // acc_empty was signalled above
        }
        if (!normed) {
#pragma unroll 1
          for (int cc = 0; cc < H3S_HEAD_DIM / 32; ++cc) {
            uint32_t acc[32];
            H3S_TMEM_LD32(tmem_base + lane_addr + a * kGemmN + gi * H3S_HEAD_DIM + cc * 32, acc);
            ptx::tmem_wait_ld();
            const int col0 = group_col0 + cc * 32;
            if (row_ok && group_ok) {
              __nv_bfloat16 *dst = prm.out + group * prm.out_stride_head + static_cast<int64_t>(row) * H3S_HEAD_DIM + cc * 32;
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 w;
                uint32_t *wp = reinterpret_cast<uint32_t *>(&w);
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                  // acc * (row_scale * column_scale), the product of the scales first (fused_qkv.py:222,424)
                  const float y0 = __fmul_rn(static_cast<float>(static_cast<int>(acc[i + e])), __fmul_rn(xs, __ldg(prm.w_scale + col0 + i + e)));
                  const float y1 = __fmul_rn(static_cast<float>(static_cast<int>(acc[i + e + 1])), __fmul_rn(xs, __ldg(prm.w_scale + col0 + i + e + 1)));
                  const __nv_bfloat162 t = __floats2bfloat162_rn(y0, y1);
                  wp[e >> 1] = *reinterpret_cast<const uint32_t *>(&t);
                }
                *reinterpret_cast<uint4 *>(dst + i) = w;
              }
            }
          }
        } else {
          // Q or K head: the whole 128-channel row of this thread is needed at once
          uint32_t y[H3S_HEAD_DIM / 2];
#pragma unroll
          for (int cc = 0; cc < H3S_HEAD_DIM / 32; ++cc) {
            uint32_t acc[32];
            H3S_TMEM_LD32(tmem_base + lane_addr + a * kGemmN + gi * H3S_HEAD_DIM + cc * 32, acc);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float2 ws = __ldg(reinterpret_cast<const float2 *>(prm.w_scale + group_col0 + cc * 32 + i));
              y[cc * 16 + (i >> 1)] =
                  pack_bf16x2(__fmul_rn(static_cast<float>(static_cast<int>(acc[i])), __fmul_rn(xs, ws.x)),
                              __fmul_rn(static_cast<float>(static_cast<int>(acc[i + 1])), __fmul_rn(xs, ws.y)));
            }
          }
          if (row_ok && group_ok) {
            const void *rope_row = nullptr;
            if (prm.rope != nullptr) {
              const int64_t offset = static_cast<int64_t>(row) * prm.rope_stride_seq;
              rope_row = prm.rope_dtype == H3S_F32
                             ? static_cast<const void *>(static_cast<const float *>(prm.rope) + offset)
                             : static_cast<const void *>(static_cast<const __nv_bfloat16 *>(prm.rope) + offset);
            }
            norm_rope_row(y, group < prm.heads ? prm.q_norm : prm.k_norm, prm.epsilon, rope_row, prm.rope_dtype,
                          prm.rope_stride_dim, prm.rope_stride_rot, prm.rope_stride_pair);
            __nv_bfloat16 *dst = prm.out + group * prm.out_stride_head + static_cast<int64_t>(row) * H3S_HEAD_DIM;
#pragma unroll
            for (int i = 0; i < H3S_HEAD_DIM / 2; i += 4)
              *reinterpret_cast<uint4 *>(dst + 2 * i) = make_uint4(y[i], y[i + 1], y[i + 2], y[i + 3]);
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&sh.acc_empty[a]);
    }
  }

  __syncthreads();
  const int code = sh.abort_word;
  if (code != 0) {
    __nanosleep(200000);
    if (threadIdx.x == 0 && prm.status != nullptr) {
      if (atomicCAS(prm.status, 0, code) == 0) prm.status[1] = blockIdx.x;
    }
  }
  if (warp == 5) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kGemmTmemCols);
  }
}

inline int make_tensor_map_u8_2d(CUtensorMap *map, const void *base, uint64_t dim0, uint64_t dim1,
                                 uint64_t stride1_bytes, uint32_t box0, uint32_t box1, const char *what) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail(H3S_ECUDA, "%s: cuTensorMapEncodeTiled is unavailable", what);
  const cuuint64_t dims[2] = {dim0, dim1};
  const cuuint64_t strides[1] = {stride1_bytes};
  const cuuint32_t box[2] = {box0, box1};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return fail(H3S_ECUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, static_cast<int>(rc));
  return H3S_OK;
}

}  // namespace h3s

extern "C" {

int h3s_convrot_quant_rows(const void *x, int64_t x_stride_row, int rows, int hidden, int8_t *x_i8,
                           float *x_scale, h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(x != nullptr && x_i8 != nullptr && x_scale != nullptr, "convrot_quant_rows: NULL pointer");
  H3S_CHECK_ARG(rows > 0 && hidden > 0 && hidden % kRotGroup == 0 && hidden / kRotGroup <= 32,
                "convrot_quant_rows: hidden %d must be a multiple of 256 and at most 8192", hidden);
  H3S_CHECK_ARG((reinterpret_cast<uintptr_t>(x) & 15) == 0 && x_stride_row % 8 == 0 && x_stride_row >= hidden,
                "convrot_quant_rows: input must be 16-byte aligned with a row stride that is a multiple of 8");
  H3S_CHECK_ARG((reinterpret_cast<uintptr_t>(x_i8) & 7) == 0, "convrot_quant_rows: output must be 8-byte aligned");
  const int groups = hidden / kRotGroup;
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  convrot_quant_rows_kernel<<<grid, groups * 32, groups * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16 *>(x), x_stride_row, rows, hidden, x_i8, x_scale);
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

static int qkv_gemm_chunk_impl(const int8_t *x_i8, const float *x_scale, const int8_t *w_i8, const float *w_scale,
                               int rows, int hidden, int n_out, void *out_bf16, int64_t out_stride_head,
                               const float *q_norm, const float *k_norm, float epsilon, const void *rope,
                               int rope_dtype, const int64_t *rope_strides, int heads, int32_t *status,
                               h3s_stream_t stream, const char *who, const h3s_qkv_carriers *carriers = nullptr) {
  using namespace h3s;
  H3S_CHECK_ARG(x_i8 && x_scale && w_i8 && w_scale && (out_bf16 || carriers), "%s: NULL pointer", who);
  H3S_CHECK_ARG(rows > 0 && hidden > 0 && hidden % kGemmK == 0, "%s: hidden %d must be a positive multiple of 128", who, hidden);
  H3S_CHECK_ARG(n_out > 0 && n_out % H3S_HEAD_DIM == 0, "%s: n_out %d must be a multiple of 128", who, n_out);
  H3S_CHECK_ARG(carriers != nullptr ||
                    (out_stride_head >= static_cast<int64_t>(rows) * H3S_HEAD_DIM && out_stride_head % 8 == 0),
                "%s: out_stride_head %lld is smaller than rows*128", who, static_cast<long long>(out_stride_head));
  H3S_CHECK_ARG(((reinterpret_cast<uintptr_t>(x_i8) | reinterpret_cast<uintptr_t>(w_i8) | reinterpret_cast<uintptr_t>(out_bf16)) & 15) == 0,
                "%s: operands must be 16-byte aligned", who);
  if (carriers != nullptr) {
    const h3s_qkv_carriers &c = *carriers;
    H3S_CHECK_ARG(heads > 0 && n_out == 3 * heads * H3S_HEAD_DIM, "%s: n_out %d is not 3*heads*128 for %d heads", who, n_out, heads);
    H3S_CHECK_ARG(c.q8 && c.q_scale && c.q_summary && c.k_summary && c.v_stage && c.stats,
                  "%s: q8, q_scale, q_summary, k_summary, v_stage and stats are required", who);
    H3S_CHECK_ARG((c.k8 != nullptr) == (c.k_scale != nullptr) && (c.k8 != nullptr) != (c.k_stage != nullptr),
                  "%s: give either k8 + k_scale (K quantised per chunk) or k_stage (K staged for smoothing)", who);
    H3S_CHECK_ARG(c.summary_dtype >= H3S_F32 && c.summary_dtype <= H3S_F64, "%s: bad summary dtype %d", who, c.summary_dtype);
    H3S_CHECK_ARG(c.row_start >= 0 && c.row_start % H3S_Q_TILE == 0 && c.row_start + rows <= c.sequence_total,
                  "%s: chunk [%d,%d) must start on a multiple of 128 inside the sequence of %d", who, c.row_start,
                  c.row_start + rows, c.sequence_total);
    H3S_CHECK_ARG(rows % H3S_Q_TILE == 0 || c.row_start + rows == c.sequence_total,
                  "%s: only the final chunk may contain a partial tile", who);
    const uintptr_t all = reinterpret_cast<uintptr_t>(c.q8) | reinterpret_cast<uintptr_t>(c.k8) |
                          reinterpret_cast<uintptr_t>(c.k_stage) | reinterpret_cast<uintptr_t>(c.v_stage);
    H3S_CHECK_ARG((all & 15) == 0 && (reinterpret_cast<uintptr_t>(c.stats) & 7) == 0,
                  "%s: carriers and staging must be 16-byte aligned, stats 8-byte aligned", who);
  }
  if (q_norm != nullptr || k_norm != nullptr || rope != nullptr) {
    H3S_CHECK_ARG(q_norm != nullptr && k_norm != nullptr, "%s: both norm weights are needed", who);
    H3S_CHECK_ARG(heads > 0 && n_out == 3 * heads * H3S_HEAD_DIM, "%s: n_out %d is not 3*heads*128 for %d heads", who, n_out, heads);
    H3S_CHECK_ARG(epsilon >= 0.f, "%s: negative epsilon", who);
    if (rope != nullptr) {
      H3S_CHECK_ARG(rope_strides != nullptr, "%s: rope strides missing", who);
      H3S_CHECK_ARG(rope_dtype == H3S_F32 || rope_dtype == H3S_BF16, "%s: rope must be fp32 or bf16", who);
    }
  }
  const int cap = h3s_device_capability();
  if (cap < 0) return cap;
  if (cap / 10 != 10) return fail(H3S_EARCH, "%s: needs an sm_100 device, found sm_%d", who, cap);
  CUtensorMap ma, mb;
  int rc = make_tensor_map_u8_2d(&ma, x_i8, hidden, rows, hidden, kGemmK, kGemmM, "qkv_gemm_chunk A map");
  if (rc) return rc;
  rc = make_tensor_map_u8_2d(&mb, w_i8, hidden, n_out, hidden, kGemmK, kGemmN, "qkv_gemm_chunk B map");
  if (rc) return rc;
  GemmParams prm;
  prm.x_scale = x_scale; prm.w_scale = w_scale; prm.out = static_cast<__nv_bfloat16 *>(out_bf16);
  prm.out_stride_head = out_stride_head; prm.status = status;
  prm.rows = rows; prm.n_out = n_out; prm.hidden = hidden;
  prm.m_tiles = ceil_div(rows, kGemmM); prm.n_tiles = ceil_div(n_out, kGemmN);
  prm.n_step = 1;
  if (carriers != nullptr) {
    auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
    int step = prm.n_tiles / 3 + 1;
    while (step > 1 && gcd(step, prm.n_tiles) != 1) --step;
    prm.n_step = step;
  }
  prm.q_norm = q_norm; prm.k_norm = k_norm; prm.rope = rope; prm.rope_dtype = rope_dtype;
  prm.rope_stride_seq = rope ? rope_strides[0] : 0; prm.rope_stride_dim = rope ? rope_strides[1] : 0;
  prm.rope_stride_rot = rope ? rope_strides[2] : 0; prm.rope_stride_pair = rope ? rope_strides[3] : 0;
  prm.heads = heads; prm.epsilon = epsilon;
  prm.wait_budget_ns = wait_budget_ns();
  prm.q8 = prm.k8 = nullptr; prm.q_scale = prm.k_scale = nullptr; prm.q_summary = prm.k_summary = nullptr;
  prm.k_stage = prm.v_stage = nullptr; prm.k_sum = nullptr; prm.v_amax_bits = nullptr;
  prm.summary_dtype = H3S_F32; prm.sequence_total = rows; prm.row_start = 0;
  prm.operand_kind = H3S_GEMM_I8; prm.row_scale = nullptr; prm.col_scale = nullptr; prm.bias = nullptr;
  prm.activation = H3S_ACT_NONE; prm.dense_out = nullptr; prm.ldc = 0;
  if (carriers != nullptr) {
    const h3s_qkv_carriers &c = *carriers;
    prm.q8 = c.q8; prm.k8 = c.k8; prm.q_scale = c.q_scale; prm.k_scale = c.k_scale;
    prm.q_summary = c.q_summary; prm.k_summary = c.k_summary;
    prm.k_stage = static_cast<__nv_bfloat16 *>(c.k_stage); prm.v_stage = static_cast<__nv_bfloat16 *>(c.v_stage);
    // statistics scratch: double k_sum[heads*128]; uint32 v_amax_bits[heads*128] (the layout of h3s_column_stats)
    double *sums = static_cast<double *>(c.stats);
    prm.k_sum = c.k_stage != nullptr ? sums : nullptr;
    prm.v_amax_bits = reinterpret_cast<unsigned int *>(sums + heads * H3S_HEAD_DIM);
    prm.summary_dtype = c.summary_dtype; prm.sequence_total = c.sequence_total; prm.row_start = c.row_start;
  }
  int device = 0, sms = 0;
  H3S_CHECK_CUDA(cudaGetDevice(&device));
  H3S_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  const int tiles = prm.m_tiles * prm.n_tiles;
  const int grid = tiles < sms ? tiles : sms;
  if (carriers != nullptr) {
    H3S_CHECK_CUDA(cudaFuncSetAttribute(qkv_gemm_kernel<kModeCarriers>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(GemmLayout<kModeCarriers>::kBytes)));
    qkv_gemm_kernel<kModeCarriers><<<grid, kGemmThreads, GemmLayout<kModeCarriers>::kBytes, static_cast<cudaStream_t>(stream)>>>(ma, mb, prm);
  } else {
    H3S_CHECK_CUDA(cudaFuncSetAttribute(qkv_gemm_kernel<kModeStaging>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(GemmLayout<kModeStaging>::kBytes)));
    qkv_gemm_kernel<kModeStaging><<<grid, kGemmThreads, GemmLayout<kModeStaging>::kBytes, static_cast<cudaStream_t>(stream)>>>(ma, mb, prm);
  }
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

int h3s_qkv_gemm_chunk(const int8_t *x_i8, const float *x_scale, const int8_t *w_i8, const float *w_scale,
                       int rows, int hidden, int n_out, void *out_bf16, int64_t out_stride_head,
                       int32_t *status, h3s_stream_t stream) {
  return qkv_gemm_chunk_impl(x_i8, x_scale, w_i8, w_scale, rows, hidden, n_out, out_bf16, out_stride_head, nullptr,
                             nullptr, 0.f, nullptr, H3S_F32, nullptr, 0, status, stream, "qkv_gemm_chunk");
}

int h3s_qkv_gemm_chunk_norm_rope(const int8_t *x_i8, const float *x_scale, const int8_t *w_i8,
                                 const float *w_scale, int rows, int hidden, int heads, void *out_bf16,
                                 int64_t out_stride_head, const float *q_norm, const float *k_norm,
                                 float epsilon, const void *rope, int rope_dtype, const int64_t *rope_strides,
                                 int32_t *status, h3s_stream_t stream) {
  H3S_CHECK_ARG(q_norm != nullptr && k_norm != nullptr, "qkv_gemm_chunk_norm_rope: NULL norm weight");
  return qkv_gemm_chunk_impl(x_i8, x_scale, w_i8, w_scale, rows, hidden, 3 * heads * H3S_HEAD_DIM, out_bf16,
                             out_stride_head, q_norm, k_norm, epsilon, rope, rope_dtype, rope_strides, heads, status,
                             stream, "qkv_gemm_chunk_norm_rope");
}

int h3s_dense_gemm(const void *a, int64_t lda_bytes, const void *b, int64_t ldb_bytes, int operand_kind, int rows,
                   int n_out, int k_bytes, const float *row_scale, const float *col_scale, const float *bias,
                   int activation, void *out_bf16, int64_t ldc, int32_t *status, h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(a != nullptr && b != nullptr && out_bf16 != nullptr, "dense_gemm: NULL pointer");
  H3S_CHECK_ARG(operand_kind >= H3S_GEMM_I8 && operand_kind <= H3S_GEMM_E4M3, "dense_gemm: unknown operand kind %d", operand_kind);
  H3S_CHECK_ARG(activation == H3S_ACT_NONE || activation == H3S_ACT_GELU_TANH, "dense_gemm: unknown activation %d", activation);
  H3S_CHECK_ARG(rows > 0 && n_out > 0 && n_out % 8 == 0, "dense_gemm: rows %d, n_out %d (a positive multiple of 8)", rows, n_out);
  H3S_CHECK_ARG(k_bytes > 0 && k_bytes % kGemmK == 0, "dense_gemm: the reduction length %d bytes must be a positive multiple of 128", k_bytes);
  H3S_CHECK_ARG(lda_bytes >= k_bytes && ldb_bytes >= k_bytes && lda_bytes % 16 == 0 && ldb_bytes % 16 == 0,
                "dense_gemm: operand row strides must be multiples of 16 bytes and cover the reduction length");
  H3S_CHECK_ARG(ldc >= n_out && ldc % 8 == 0, "dense_gemm: ldc %lld must be a multiple of 8 and at least n_out", static_cast<long long>(ldc));
  H3S_CHECK_ARG(((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out_bf16)) & 15) == 0,
                "dense_gemm: operands and output must be 16-byte aligned");
  const int cap = h3s_device_capability();
  if (cap < 0) return cap;
  if (cap / 10 != 10) return fail(H3S_EARCH, "dense_gemm: needs an sm_100 device, found sm_%d", cap);
  CUtensorMap ma, mb;
  int rc = make_tensor_map_u8_2d(&ma, a, k_bytes, rows, lda_bytes, kGemmK, kGemmM, "dense_gemm A map");
  if (rc) return rc;
  rc = make_tensor_map_u8_2d(&mb, b, k_bytes, n_out, ldb_bytes, kGemmK, kGemmN, "dense_gemm B map");
  if (rc) return rc;
  GemmParams prm;
  memset(&prm, 0, sizeof(prm));
  prm.x_scale = row_scale; prm.status = status;
  prm.rows = rows; prm.n_out = n_out; prm.hidden = k_bytes;
  prm.m_tiles = ceil_div(rows, kGemmM); prm.n_tiles = ceil_div(n_out, kGemmN); prm.n_step = 1;
  prm.heads = 1; prm.wait_budget_ns = wait_budget_ns();
  prm.operand_kind = operand_kind; prm.row_scale = row_scale; prm.col_scale = col_scale; prm.bias = bias;
  prm.activation = activation; prm.dense_out = static_cast<__nv_bfloat16 *>(out_bf16); prm.ldc = ldc;
  int device = 0, sms = 0;
  H3S_CHECK_CUDA(cudaGetDevice(&device));
  H3S_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  H3S_CHECK_CUDA(cudaFuncSetAttribute(qkv_gemm_kernel<kModeDense>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(GemmLayout<kModeDense>::kBytes)));
  const int tiles = prm.m_tiles * prm.n_tiles;
  qkv_gemm_kernel<kModeDense><<<tiles < sms ? tiles : sms, kGemmThreads, GemmLayout<kModeDense>::kBytes,
                               static_cast<cudaStream_t>(stream)>>>(ma, mb, prm);
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

int h3s_qkv_gemm_chunk_carriers(const int8_t *x_i8, const float *x_scale, const int8_t *w_i8,
                                const float *w_scale, int rows, int hidden, int heads,
                                const h3s_qkv_carriers *carriers, const float *q_norm, const float *k_norm,
                                float epsilon, const void *rope, int rope_dtype, const int64_t *rope_strides,
                                int32_t *status, h3s_stream_t stream) {
  H3S_CHECK_ARG(carriers != nullptr, "qkv_gemm_chunk_carriers: NULL carrier description");
  return qkv_gemm_chunk_impl(x_i8, x_scale, w_i8, w_scale, rows, hidden, 3 * heads * H3S_HEAD_DIM, nullptr, 0, q_norm,
                             k_norm, epsilon, rope, rope_dtype, rope_strides, heads, status, stream,
                             "qkv_gemm_chunk_carriers", carriers);
}

}  // extern "C"
