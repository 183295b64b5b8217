// Block-sparse attention on the INT8 Q/K + FP8 V carriers for sm_100a.
//
// One CTA owns one 128-row query tile of one head and walks that tile's list
// of 64-row KV tiles:
//   S = Q8 . K8^T      tcgen05.mma kind::i8, 128x64x128, int32 in TMEM (2 buffers)
//   P = exp2(c*S - m)  FP32 in registers, one thread per query row, m an integer
//                      so every rescale is an exact power of two
//   O += P8 . V8       tcgen05.mma kind::f8f6f4, 128x128x64, fp32 in TMEM
// P is carried as two E4M3 terms (hi = P truncated to 4 significant bits,
// lo = E4M3(P - hi)) and the product is issued once per term, which gives the
// probabilities ~7 significant bits; a single-term mode (flag
// H3S_ATTN_P_SINGLE) trades that precision for fewer MMAs.
// Warp roles: warps 0-3 softmax/epilogue (TMEM lanes 32w..32w+31), warp 4
// TMA producer (K tile + V^T tile per stage, only the listed tiles are ever
// fetched), warp 5 MMA issuer and TMEM owner.  Two CTAs share an SM
// (2 x 256 TMEM columns, 2 x ~98 KB shared memory), so one CTA's softmax
// overlaps the other's MMAs.
//
// O is rescaled lazily: the reference point m is only raised when a score
// exceeds it by more than 8.75 (P then stays <= 2^8.75 = 431 < 448 = E4M3 max).
#include <climits>

#include "common.cuh"
#include "ptx.cuh"
#include "tma.cuh"

namespace h3s {

constexpr int kStages = 5;
constexpr int kAttnThreads = 192;
constexpr int kTmemCols = 256;
constexpr uint32_t kQBytes = H3S_Q_TILE * H3S_HEAD_DIM;        // 16384
constexpr uint32_t kKBytes = H3S_KV_TILE * H3S_HEAD_DIM;       // 8192
constexpr uint32_t kVBytes = H3S_HEAD_DIM * H3S_KV_TILE;       // 8192
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + kQBytes;
constexpr uint32_t kOffV = kOffK + kStages * kKBytes;
constexpr uint32_t kOffBar = kOffV + kStages * kVBytes;  // P lives in TMEM, not in shared memory
constexpr uint32_t kAttnSmemBytes = kOffBar + 1024 + 1024;  // barriers/scalars + alignment slack
// P = exp2(logit - m) with m = ceil(rowmax) - kPOffset when m is (re)set, so the
// largest probability starts in (64, 128]; m is raised again only when a score
// would push P past 2^8.75 (E4M3 max 448).  FP8 reaches down to 2^-9/2^-10, so
// keys more than 17-18 bits below the row maximum drop out of the numerator (they
// stay in the FP32 row sum); with the reference point 5 bits below the maximum
// instead of 7 a 76k-key row lost up to 6.5 % of its mass that way, now 2.5 %,
// for ~2 % more time spent rescaling.
constexpr float kRescaleThreshold = 8.75f;
constexpr float kPOffset = 7.0f;
constexpr float kIntBias = 12582912.0f;  // 1.5 * 2^23: float(kIntBias + s) has bits 0x4b400000 + s

enum AbortCode {
  kAbortQFull = 1, kAbortKvFull, kAbortKvEmpty, kAbortSFull, kAbortPFull, kAbortPEmpty,
  kAbortPvDone, kAbortFinal
};

struct AttnParams {
  const float *q_scale;
  const float *k_scale;
  const float *v_scale;
  const int32_t *route;  // (heads, q_stop-q_start, route_len) or null
  void *out;
  int32_t *status;
  int64_t out_stride_h, out_stride_s;
  int route_len, q_start, q_stop;
  int heads, sequence, q_tiles, kv_tiles;
  int out_dtype;
  // head-sharded runs: every output tile is also stored into these buffers
  // (the same slice of each peer GPU's full output, reached over NVLink with
  // plain stores), so no separate gather pass is needed
  void *peer_out[H3S_MAX_PEER_OUTPUTS];
  int n_peer_out;
  // Bound of the waits for TMA loads; a wait further down the pipeline (QK^T
  // result 2x, P 3x, P.V and free stages 4x) gets a multiple, so that when a
  // stage stalls the wait closest to the cause is the one that runs out first
  // and names it in the status words.
  unsigned long long wait_budget_ns;
  // self-test of the bounded waits (H3S_ATTN_TEST_DROP_KV_LOAD): the producer
  // never issues the K/V load of this iteration, so the wait for it runs out
  int drop_kv_load;                   // iteration index, -1 = none
};

struct AttnShared {
  uint64_t q_full;
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t p_empty[2];
  uint32_t tmem_base;
  int abort_word;
  int tile_index[kStages];    // KV tile held by each stage ...
  float tile_scale[kStages];  // ... and its k_scale, written by the producer
  float v_scale[H3S_HEAD_DIM];
};
static_assert(sizeof(AttnShared) <= 1024, "barrier block too large");

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Every lane polls the barrier; the warp then agrees on the outcome so that
// the .sync.aligned tcgen05 instructions that follow stay convergent even if
// the abort word was raised between two lanes' polls.
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity, volatile int *abort_word, int code,
                                          unsigned long long budget_ns) {
  const bool ok = ptx::mbar_wait(bar, parity, abort_word, code, budget_ns);
  return __all_sync(0xffffffffu, ok);
}

// packed fp32x2 arithmetic (one instruction for two lanes of a 64-bit register pair)
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<unsigned long long &>(d))
      : "l"(reinterpret_cast<unsigned long long &>(a)), "l"(reinterpret_cast<unsigned long long &>(b)),
        "l"(reinterpret_cast<unsigned long long &>(c)));
  return d;
}

__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("mul.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long &>(d))
      : "l"(reinterpret_cast<unsigned long long &>(a)), "l"(reinterpret_cast<unsigned long long &>(b)));
  return d;
}

__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("add.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long &>(d))
      : "l"(reinterpret_cast<unsigned long long &>(a)), "l"(reinterpret_cast<unsigned long long &>(b)));
  return d;
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// Constants of one tile's exponentials: x = c*f + bias (f carries the 1.5*2^23 offset).
struct ExpArgs {
  float2 c2, bias2;
};

// The int32 scores become fp32 without a conversion instruction: for |s| < 2^22,
// bits(12582912.0f) + s are the bits of the float 12582912 + s exactly, and the
// offset is folded into the constants of the FMA that follows.
// kRagged (last KV tile of a sequence that is not a multiple of 64): keys from
// n_valid on are masked, P = 0.
template <bool kTwoTerm, bool kRagged>
__device__ __forceinline__ float exp_and_pack(const uint32_t (&s)[64], const ExpArgs &a, int n_valid,
                                              uint32_t (&packed)[16], uint32_t (&packed_lo)[16]) {
  const float2 minus1 = make_float2(-1.f, -1.f);
  float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 64; i += 4) {
    float f[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      f[k] = __uint_as_float(s[i + k] + 0x4b400000u);
      if (kRagged && i + k >= n_valid) f[k] = -INFINITY;
    }
    const float2 x01 = fma2(a.c2, make_float2(f[0], f[1]), a.bias2);
    const float2 x23 = fma2(a.c2, make_float2(f[2], f[3]), a.bias2);
    const float2 p01 = make_float2(fast_exp2(x01.x), fast_exp2(x01.y));
    const float2 p23 = make_float2(fast_exp2(x23.x), fast_exp2(x23.y));
    sum2 = add2(sum2, p01);
    sum2 = add2(sum2, p23);
    if (kTwoTerm) {
      const float2 h01 = make_float2(__uint_as_float(__float_as_uint(p01.x) & 0xfff00000u),
                                     __uint_as_float(__float_as_uint(p01.y) & 0xfff00000u));
      const float2 h23 = make_float2(__uint_as_float(__float_as_uint(p23.x) & 0xfff00000u),
                                     __uint_as_float(__float_as_uint(p23.y) & 0xfff00000u));
      const float2 r01 = fma2(h01, minus1, p01);
      const float2 r23 = fma2(h23, minus1, p23);
      packed[i >> 2] = pack_e4m3x4(h01.x, h01.y, h23.x, h23.y);
      packed_lo[i >> 2] = pack_e4m3x4(r01.x, r01.y, r23.x, r23.y);
    } else {
      packed[i >> 2] = pack_e4m3x4(p01.x, p01.y, p23.x, p23.y);
    }
  }
  return sum2.x + sum2.y;
}

template <typename OutT> __device__ __forceinline__ void store_out8(OutT *dst, const float (&v)[8]);
template <> __device__ __forceinline__ void store_out8<float>(float *dst, const float (&v)[8]) {
  reinterpret_cast<float4 *>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4 *>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store_out8<__nv_bfloat16>(__nv_bfloat16 *dst, const float (&v)[8]) {
  uint4 w;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(v[0], v[1]); w.x = *reinterpret_cast<uint32_t *>(&t);
  t = __floats2bfloat162_rn(v[2], v[3]); w.y = *reinterpret_cast<uint32_t *>(&t);
  t = __floats2bfloat162_rn(v[4], v[5]); w.z = *reinterpret_cast<uint32_t *>(&t);
  t = __floats2bfloat162_rn(v[6], v[7]); w.w = *reinterpret_cast<uint32_t *>(&t);
  *reinterpret_cast<uint4 *>(dst) = w;
}
template <> __device__ __forceinline__ void store_out8<__half>(__half *dst, const float (&v)[8]) {
  uint4 w;
  __half2 t;
  t = __floats2half2_rn(v[0], v[1]); w.x = *reinterpret_cast<uint32_t *>(&t);
  t = __floats2half2_rn(v[2], v[3]); w.y = *reinterpret_cast<uint32_t *>(&t);
  t = __floats2half2_rn(v[4], v[5]); w.z = *reinterpret_cast<uint32_t *>(&t);
  t = __floats2half2_rn(v[6], v[7]); w.w = *reinterpret_cast<uint32_t *>(&t);
  *reinterpret_cast<uint4 *>(dst) = w;
}

template <typename OutT, bool kSplitP>
__global__ void __launch_bounds__(kAttnThreads, 2)
sparse_attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const AttnParams prm) {
  extern __shared__ unsigned char smem_dyn[];
  // SWIZZLE_128B tiles need 1024-byte alignment
  unsigned char *smem = reinterpret_cast<unsigned char *>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
  AttnShared &sh = *reinterpret_cast<AttnShared *>(smem + kOffBar);
  volatile int *abort_word = &sh.abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- work item: dense (long) rows first, then the routed rows ----
  const int n_sparse = prm.route != nullptr ? prm.q_stop - prm.q_start : 0;
  const int n_dense = prm.q_tiles - n_sparse;
  int head, tq;
  bool dense;
  {
    const int w = blockIdx.x;
    const int dense_items = prm.heads * n_dense;
    if (w < dense_items) {
      dense = true;
      head = w / n_dense;
      const int i = w - head * n_dense;
      tq = (n_sparse == 0 || i < prm.q_start) ? i : prm.q_stop + (i - prm.q_start);
    } else {
      dense = false;
      const int v = w - dense_items;
      head = v / n_sparse;
      tq = prm.q_start + (v - head * n_sparse);
    }
  }
  const int n_iter = dense ? prm.kv_tiles : prm.route_len;
  const int32_t *route_row =
      dense ? nullptr
            : prm.route + (static_cast<int64_t>(head) * n_sparse + (tq - prm.q_start)) * prm.route_len;

  // ---- setup ----
  if (threadIdx.x == 0) {
    ptx::mbar_init(&sh.q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&sh.kv_full[i], 1);
      ptx::mbar_init(&sh.kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&sh.s_full[i], 1);
      ptx::mbar_init(&sh.p_full[i], 4);
      ptx::mbar_init(&sh.p_empty[i], 1);
    }
    sh.abort_word = 0;
    ptx::fence_mbar_init();
  }
  if (threadIdx.x < H3S_HEAD_DIM) sh.v_scale[threadIdx.x] = __ldg(prm.v_scale + head * H3S_HEAD_DIM + threadIdx.x);
  if (warp == 5) {
    ptx::tmem_alloc(&sh.tmem_base, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;
  const uint32_t tmem_s = tmem_base;          // 2 x 64 columns, int32
  const uint32_t tmem_o = tmem_base + 128;    // 128 columns, fp32

  if (warp == 4) {
    // =================== TMA producer ===================
    // The whole warp fetches the tile indices and K scales of 32 tiles at a
    // time (two dependent global loads, kept off everybody's critical path);
    // lane 0 then feeds the stage ring and leaves each stage's index and scale
    // in shared memory for the softmax warps.
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_q);
      ptx::prefetch_tensormap(&map_k);
      ptx::prefetch_tensormap(&map_v);
      ptx::mbar_arrive_expect_tx(&sh.q_full, kQBytes);
      ptx::tma_load_3d(smem + kOffQ, &map_q, &sh.q_full, 0, tq * H3S_Q_TILE, head);
    }
    const float *k_scale = prm.k_scale + static_cast<int64_t>(head) * prm.kv_tiles;
    bool ok = true;
    for (int j0 = 0; ok && j0 < n_iter; j0 += 32) {
      const int mine = min(j0 + lane, n_iter - 1);
      const int my_tile = dense ? mine : __ldg(route_row + mine);
      const float my_scale = __ldg(k_scale + my_tile);
      const int batch = min(32, n_iter - j0);
      for (int i = 0; i < batch; ++i) {
        const int t = __shfl_sync(0xffffffffu, my_tile, i);
        const float ks = __shfl_sync(0xffffffffu, my_scale, i);
        if (lane == 0) {
          const int j = j0 + i;
          const int s = j % kStages;
          const uint32_t use = static_cast<uint32_t>(j / kStages);
          ok = ptx::mbar_wait(&sh.kv_empty[s], (use & 1u) ^ 1u, abort_word, kAbortKvEmpty, 4 * prm.wait_budget_ns);
          if (ok && j != prm.drop_kv_load) {
            sh.tile_index[s] = t;
            sh.tile_scale[s] = ks;
            ptx::mbar_arrive_expect_tx(&sh.kv_full[s], kKBytes + kVBytes);
            ptx::tma_load_3d(smem + kOffK + s * kKBytes, &map_k, &sh.kv_full[s], 0, t * H3S_KV_TILE, head);
            ptx::tma_load_3d(smem + kOffV + s * kVBytes, &map_v, &sh.kv_full[s], t * H3S_KV_TILE, 0, head);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
      }
    }
  } else if (warp == 5) {
    // =================== MMA issuer ===================
    {
      constexpr uint32_t idesc_qk = ptx::umma_idesc(2, 1, 1, H3S_Q_TILE, H3S_KV_TILE);
      constexpr uint32_t idesc_pv = ptx::umma_idesc(1, 0, 0, H3S_Q_TILE, H3S_HEAD_DIM);
      const uint64_t q_desc = ptx::umma_desc_kmajor(ptx::smem_u32(smem + kOffQ), 1024, ptx::kSwizzle128);
      const uint64_t k_desc0 = ptx::umma_desc_kmajor(ptx::smem_u32(smem + kOffK), 1024, ptx::kSwizzle128);
      const uint64_t v_desc0 = ptx::umma_desc_kmajor(ptx::smem_u32(smem + kOffV), 512, ptx::kSwizzle64);
      auto issue_qk = [&](int j) {
        if (ptx::elect_one()) {
          const uint64_t k_desc = k_desc0 + static_cast<uint64_t>((j % kStages) * (kKBytes >> 4));
#pragma unroll
          for (int k = 0; k < H3S_HEAD_DIM / 32; ++k)
            ptx::umma_i8(tmem_s + (j & 1) * H3S_KV_TILE, q_desc + 2 * k, k_desc + 2 * k, idesc_qk, k > 0);
          ptx::tc_commit(&sh.s_full[j & 1]);
        }
        __syncwarp();
      };
      auto wait_stage = [&](int j) {
        return warp_wait(&sh.kv_full[j % kStages], static_cast<uint32_t>(j / kStages) & 1u, abort_word,
                         kAbortKvFull, prm.wait_budget_ns);
      };
      bool ok = warp_wait(&sh.q_full, 0, abort_word, kAbortQFull, prm.wait_budget_ns);
      for (int j = 0; ok && j < min(2, n_iter); ++j) {
        ok = wait_stage(j);
        if (ok) {
          ptx::tc_fence_after();
          issue_qk(j);
        }
      }
      for (int i = 0; ok && i < n_iter; ++i) {
        const int s = i % kStages, b = i & 1;
        if (i + 2 < n_iter && !wait_stage(i + 2)) { ok = false; break; }
        if (!warp_wait(&sh.p_full[b], static_cast<uint32_t>(i >> 1) & 1u, abort_word, kAbortPFull, 3 * prm.wait_budget_ns)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        if (ptx::elect_one()) {
          const uint64_t v_desc = v_desc0 + static_cast<uint64_t>(s * (kVBytes >> 4));
#pragma unroll
          for (int k = 0; k < H3S_KV_TILE / 32; ++k)
            ptx::umma_f8_ts(tmem_o, tmem_s + b * H3S_KV_TILE + k * 8, v_desc + 2 * k, idesc_pv,
                            (i > 0 || k > 0) ? 1u : 0u);
          if (kSplitP) {
#pragma unroll
            for (int k = 0; k < H3S_KV_TILE / 32; ++k)
              ptx::umma_f8_ts(tmem_o, tmem_s + b * H3S_KV_TILE + 16 + k * 8, v_desc + 2 * k, idesc_pv, 1u);
          }
          ptx::tc_commit(&sh.kv_empty[s]);
          ptx::tc_commit(&sh.p_empty[b]);
        }
        __syncwarp();
        if (i + 2 < n_iter) issue_qk(i + 2);
      }
    }
  } else {
    // =================== softmax + epilogue (warps 0-3) ===================
    const int row = warp * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float q_scale = __ldg(prm.q_scale + head * prm.q_tiles + tq) * (0.08838834764831845f * 1.4426950408889634f);
    float m_used = -INFINITY;
    float l = 0.f;
    bool ok = true;

    for (int j = 0; j < n_iter; ++j) {
      const int b = j & 1;
      const uint32_t use = static_cast<uint32_t>(j >> 1);
      if (!warp_wait(&sh.s_full[b], use & 1u, abort_word, kAbortSFull, 2 * prm.wait_budget_ns)) { ok = false; break; }
      ptx::tc_fence_after();
      uint32_t s[64];
      H3S_TMEM_LD32(tmem_s + lane_addr + b * H3S_KV_TILE, s);
      {
        uint32_t *s_hi = s + 32;
        H3S_TMEM_LD32(tmem_s + lane_addr + b * H3S_KV_TILE + 32, s_hi);
      }
      ptx::tmem_wait_ld();

      // index and K scale of this tile, left in shared memory by the producer
      // before the stage was handed to the MMA warp (stage free only after P.V(j))
      const int t = sh.tile_index[j % kStages];
      const float c = q_scale * sh.tile_scale[j % kStages];
      const int n_valid = min(H3S_KV_TILE, prm.sequence - t * H3S_KV_TILE);

      // Keys beyond the sequence (ragged last tile only) get the most negative
      // score, which keeps them out of the maximum; the exponential loop sets
      // their P to 0.
      if (n_valid < H3S_KV_TILE) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i >= n_valid) s[i] = 0x80000000u;
      }
      // row maximum on the raw integers (3-input integer max), four independent
      // chains: a single chain of 32 dependent instructions costs more than the
      // arithmetic
      int im0 = __vimax3_s32(s[0], s[1], s[2]), im1 = __vimax3_s32(s[3], s[4], s[5]);
      int im2 = __vimax3_s32(s[6], s[7], s[8]), im3 = __vimax3_s32(s[9], s[10], s[11]);
#pragma unroll
      for (int i = 12; i + 7 < 64; i += 8) {
        im0 = __vimax3_s32(im0, s[i], s[i + 1]);
        im1 = __vimax3_s32(im1, s[i + 2], s[i + 3]);
        im2 = __vimax3_s32(im2, s[i + 4], s[i + 5]);
        im3 = __vimax3_s32(im3, s[i + 6], s[i + 7]);
      }
      im0 = __vimax3_s32(im0, s[60], s[61]);
      im1 = __vimax3_s32(im1, s[62], s[63]);
      const float fm = static_cast<float>(__vimax3_s32(im0, im1, max(im2, im3)));
      const float mx = c * fm;  // c > 0
      const bool need = mx > m_used + kRescaleThreshold;
      if (__any_sync(0xffffffffu, need)) {
        const float m_new = need ? ceilf(mx) - kPOffset : m_used;
        const float alpha = fast_exp2(m_used - m_new);  // 1 when unchanged, 0 from -inf
        if (j > 0) {
          const int pb = (j - 1) & 1;
          const uint32_t pu = static_cast<uint32_t>((j - 1) >> 1);
          if (!warp_wait(&sh.p_empty[pb], pu & 1u, abort_word, kAbortPvDone, 4 * prm.wait_budget_ns)) { ok = false; break; }
          ptx::tc_fence_after();
#pragma unroll 1
          for (int cc = 0; cc < H3S_HEAD_DIM / 32; ++cc) {
            uint32_t o[32];
            H3S_TMEM_LD32(tmem_o + lane_addr + cc * 32, o);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            H3S_TMEM_ST32(tmem_o + lane_addr + cc * 32, o);
          }
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
        }
        l *= alpha;
        m_used = m_new;
      }

      // P = exp2(c*f - m), two elements per instruction (packed fp32x2 FMA/ADD);
      // x = c*(f - 12582912) - m
      const float bias = -fmaf(c, kIntBias, m_used);
      ExpArgs args;
      args.c2 = make_float2(c, c);
      args.bias2 = make_float2(bias, bias);
      uint32_t packed[16];
      uint32_t packed_lo[16];
      // P(j) overwrites this thread's own lane of S buffer b (already in
      // registers).  The MMA that produced S(j) was issued after P.V(j-2), so
      // nothing still reads these columns.
      if (n_valid < H3S_KV_TILE) {
        l += exp_and_pack<kSplitP, true>(s, args, n_valid, packed, packed_lo);
      } else {
        l += exp_and_pack<kSplitP, false>(s, args, n_valid, packed, packed_lo);
      }
      H3S_TMEM_ST16(tmem_s + lane_addr + b * H3S_KV_TILE, packed);
      if (kSplitP) H3S_TMEM_ST16(tmem_s + lane_addr + b * H3S_KV_TILE + 16, packed_lo);
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&sh.p_full[b]);
    }

    if (ok) {
      const int last = n_iter - 1;
      ok = warp_wait(&sh.p_empty[last & 1], static_cast<uint32_t>(last >> 1) & 1u, abort_word, kAbortFinal, 4 * prm.wait_budget_ns);
    }
    if (ok) {
      // Epilogue: O * v_scale / l -> OutT, staged through shared memory (the K
      // stage ring is free: every TMA load has been consumed) so that each warp
      // writes its 32 rows as full contiguous lines to the local output.  A
      // warp only reads back the rows it staged itself, so __syncwarp is the
      // only synchronisation.  In a head-sharded run the staged tile is also
      // copied to the peers, by the whole CTA, after the teardown barrier.
      ptx::tc_fence_after();
      const float inv_l = 1.0f / l;
      constexpr int kRowBytes = H3S_HEAD_DIM * static_cast<int>(sizeof(OutT));
      constexpr int kChunksPerRow = kRowBytes / 16;
      unsigned char *stage = smem + kOffK;
      static_assert(H3S_Q_TILE * kRowBytes <= kStages * (kKBytes + kVBytes), "output tile must fit the stage ring");
      unsigned char *my_row = stage + row * kRowBytes;
#pragma unroll 1
      for (int cc = 0; cc < H3S_HEAD_DIM / 32; ++cc) {
        uint32_t o[32];
        H3S_TMEM_LD32(tmem_o + lane_addr + cc * 32, o);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            v[e] = __uint_as_float(o[i + e]) * sh.v_scale[cc * 32 + i + e] * inv_l;
          // 8 values = one (bf16/fp16) or two (fp32) 16-byte chunks; the chunk index is
          // XORed with the row so that the 32 rows of a warp do not collide on banks
          constexpr int kChunks8 = 8 * static_cast<int>(sizeof(OutT)) / 16;
          const int chunk0 = (cc * 32 + i) * static_cast<int>(sizeof(OutT)) / 16;
          __align__(16) OutT tmp[8];
          store_out8<OutT>(tmp, v);
#pragma unroll
          for (int k = 0; k < kChunks8; ++k)
            *reinterpret_cast<uint4 *>(my_row + (((chunk0 + k) ^ (row & 15)) << 4)) =
                reinterpret_cast<const uint4 *>(tmp)[k];
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      const int warp_row0 = warp * 32;
      unsigned char *base = static_cast<unsigned char *>(prm.out);
#pragma unroll 4
      for (int idx = lane; idx < 32 * kChunksPerRow; idx += 32) {
        const int r = warp_row0 + idx / kChunksPerRow, c = idx % kChunksPerRow;
        const int grow = tq * H3S_Q_TILE + r;
        if (grow < prm.sequence) {
          const uint4 value = *reinterpret_cast<const uint4 *>(stage + r * kRowBytes + ((c ^ (r & 15)) << 4));
          unsigned char *dst = base + (head * prm.out_stride_h + static_cast<int64_t>(grow) * prm.out_stride_s) *
                                          static_cast<int64_t>(sizeof(OutT)) + c * 16;
          *reinterpret_cast<uint4 *>(dst) = value;
        }
      }
    }
  }

  // ---- teardown ----
  __syncthreads();
  const int code = sh.abort_word;
  if (code != 0) {
    // leave time for copies / MMAs still in flight before releasing TMEM and shared memory
    __nanosleep(200000);
    if (threadIdx.x == 0 && prm.status != nullptr) {
      if (atomicCAS(prm.status, 0, code) == 0) {
        prm.status[1] = blockIdx.x;
        prm.status[2] = head;
        prm.status[3] = tq;
      }
    }
  }
  if (warp == 5) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  // Head-sharded run: the finished tile, still staged in shared memory, goes to
  // the same slice of every peer GPU's output with plain stores over NVLink.
  // All six warps share the copy (the producer and MMA warps have nothing left
  // to do), and each 16-byte chunk is sent to all peers back to back, so the
  // stores of one CTA are spread over every link at once instead of filling
  // one destination after the other.
  if (code == 0 && prm.n_peer_out > 0) {
    constexpr int kRowBytes = H3S_HEAD_DIM * static_cast<int>(sizeof(OutT));
    constexpr int kChunksPerRow = kRowBytes / 16;
    const unsigned char *stage = smem + kOffK;
    const int64_t tile_offset = head * prm.out_stride_h * static_cast<int64_t>(sizeof(OutT));
    for (int idx = threadIdx.x; idx < H3S_Q_TILE * kChunksPerRow; idx += kAttnThreads) {
      const int r = idx / kChunksPerRow, c = idx % kChunksPerRow;
      const int grow = tq * H3S_Q_TILE + r;
      if (grow < prm.sequence) {
        const uint4 value = *reinterpret_cast<const uint4 *>(stage + r * kRowBytes + ((c ^ (r & 15)) << 4));
        const int64_t at = tile_offset + static_cast<int64_t>(grow) * prm.out_stride_s * static_cast<int64_t>(sizeof(OutT)) + c * 16;
#pragma unroll
        for (int d = 0; d < H3S_MAX_PEER_OUTPUTS; ++d)
          if (d < prm.n_peer_out) *reinterpret_cast<uint4 *>(static_cast<unsigned char *>(prm.peer_out[d]) + at) = value;
      }
    }
  }
}

template <typename OutT, bool kSplitP>
static int launch_attn_tc_impl(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv,
                               const AttnParams &prm, cudaStream_t stream) {
  H3S_CHECK_CUDA(cudaFuncSetAttribute(sparse_attn_tc_kernel<OutT, kSplitP>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(kAttnSmemBytes)));
  const int grid = prm.heads * prm.q_tiles;
  sparse_attn_tc_kernel<OutT, kSplitP><<<grid, kAttnThreads, kAttnSmemBytes, stream>>>(mq, mk, mv, prm);
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

template <typename OutT>
static int launch_attn_tc(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv,
                          const AttnParams &prm, bool split_p, cudaStream_t stream) {
  return split_p ? launch_attn_tc_impl<OutT, true>(mq, mk, mv, prm, stream)
                 : launch_attn_tc_impl<OutT, false>(mq, mk, mv, prm, stream);
}

int check_attn_args(const int8_t *q8, const int8_t *k8, const uint8_t *v8t, const float *q_scale,
                    const float *k_scale, const float *v_scale, const int32_t *route, int route_len,
                    int q_start, int q_stop, void *out, int out_dtype, int64_t out_stride_h,
                    int64_t out_stride_s, int heads, int sequence, const char *who) {
  H3S_CHECK_ARG(q8 && k8 && v8t && q_scale && k_scale && v_scale && out, "%s: NULL pointer", who);
  H3S_CHECK_ARG(heads > 0 && sequence > 0, "%s: empty problem (heads=%d sequence=%d)", who, heads, sequence);
  H3S_CHECK_ARG(out_dtype == H3S_F32 || out_dtype == H3S_BF16 || out_dtype == H3S_F16, "%s: bad out dtype %d", who, out_dtype);
  const int vec = out_dtype == H3S_F32 ? 4 : 8;
  H3S_CHECK_ARG((reinterpret_cast<uintptr_t>(out) & 15) == 0 && out_stride_h % vec == 0 && out_stride_s % vec == 0 && out_stride_s >= H3S_HEAD_DIM,
                "%s: output must be 16-byte aligned with strides that are multiples of %d elements", who, vec);
  H3S_CHECK_ARG(((reinterpret_cast<uintptr_t>(q8) | reinterpret_cast<uintptr_t>(k8) | reinterpret_cast<uintptr_t>(v8t)) & 15) == 0,
                "%s: carriers must be 16-byte aligned", who);
  const int q_tiles = ceil_div(sequence, H3S_Q_TILE), kv_tiles = ceil_div(sequence, H3S_KV_TILE);
  if (route != nullptr) {
    H3S_CHECK_ARG(0 <= q_start && q_start < q_stop && q_stop <= q_tiles, "%s: bad routed query range [%d,%d) of %d", who, q_start, q_stop, q_tiles);
    H3S_CHECK_ARG(route_len >= 1 && route_len <= kv_tiles, "%s: route_len %d outside [1,%d]", who, route_len, kv_tiles);
  }
  return H3S_OK;
}

}  // namespace h3s

namespace h3s {
static int sparse_attn_fwd_impl(const int8_t *q8, const int8_t *k8, const uint8_t *v8t,
                                const float *q_scale, const float *k_scale, const float *v_scale,
                                const int32_t *route, int route_len, int q_start, int q_stop,
                                void *out, void *const *peer_out, int n_peer_out, int out_dtype,
                                int64_t out_stride_h, int64_t out_stride_s,
                                int heads, int sequence, int flags, int32_t *status,
                                h3s_stream_t stream) {
  H3S_CHECK_ARG(n_peer_out >= 0 && n_peer_out <= H3S_MAX_PEER_OUTPUTS && (n_peer_out == 0 || peer_out != nullptr),
                "sparse_attn_fwd: %d peer outputs (at most %d)", n_peer_out, H3S_MAX_PEER_OUTPUTS);
  for (int i = 0; i < n_peer_out; ++i)
    H3S_CHECK_ARG(peer_out[i] != nullptr && (reinterpret_cast<uintptr_t>(peer_out[i]) & 15) == 0,
                  "sparse_attn_fwd: peer output %d is NULL or not 16-byte aligned", i);
  {
    int rc = check_attn_args(q8, k8, v8t, q_scale, k_scale, v_scale, route, route_len, q_start, q_stop, out,
                             out_dtype, out_stride_h, out_stride_s, heads, sequence, "sparse_attn_fwd");
    if (rc) return rc;
  }
  const int cap = h3s_device_capability();
  if (cap < 0) return cap;
  if (cap / 10 != 10) return fail(H3S_EARCH, "sparse_attn_fwd: needs an sm_100 device, found sm_%d", cap);

  const uint64_t S = static_cast<uint64_t>(sequence);
  const uint64_t padded = static_cast<uint64_t>(ceil_div(sequence, 128)) * 128;
  CUtensorMap mq, mk, mv;
  int rc = make_tensor_map_u8_3d(&mq, q8, H3S_HEAD_DIM, S, heads, H3S_HEAD_DIM, S * H3S_HEAD_DIM,
                                 H3S_HEAD_DIM, H3S_Q_TILE, CU_TENSOR_MAP_SWIZZLE_128B, "sparse_attn_fwd Q map");
  if (rc) return rc;
  rc = make_tensor_map_u8_3d(&mk, k8, H3S_HEAD_DIM, S, heads, H3S_HEAD_DIM, S * H3S_HEAD_DIM, H3S_HEAD_DIM,
                             H3S_KV_TILE, CU_TENSOR_MAP_SWIZZLE_128B, "sparse_attn_fwd K map");
  if (rc) return rc;
  rc = make_tensor_map_u8_3d(&mv, v8t, padded, H3S_HEAD_DIM, heads, padded, padded * H3S_HEAD_DIM,
                             H3S_KV_TILE, H3S_HEAD_DIM, CU_TENSOR_MAP_SWIZZLE_64B, "sparse_attn_fwd V map");
  if (rc) return rc;

  AttnParams prm;
  prm.q_scale = q_scale; prm.k_scale = k_scale; prm.v_scale = v_scale;
  prm.route = route; prm.out = out; prm.status = status;
  prm.out_stride_h = out_stride_h; prm.out_stride_s = out_stride_s;
  prm.route_len = route_len; prm.q_start = q_start; prm.q_stop = q_stop;
  prm.heads = heads; prm.sequence = sequence;
  prm.q_tiles = ceil_div(sequence, H3S_Q_TILE); prm.kv_tiles = ceil_div(sequence, H3S_KV_TILE);
  prm.out_dtype = out_dtype;
  prm.n_peer_out = n_peer_out;
  prm.wait_budget_ns = wait_budget_ns();
  prm.drop_kv_load = (flags & H3S_ATTN_TEST_DROP_KV_LOAD) ? 0 : -1;
  for (int i = 0; i < H3S_MAX_PEER_OUTPUTS; ++i) prm.peer_out[i] = i < n_peer_out ? peer_out[i] : nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool split_p = (flags & H3S_ATTN_P_SINGLE) == 0;
  switch (out_dtype) {
    case H3S_F32: return launch_attn_tc<float>(mq, mk, mv, prm, split_p, s);
    case H3S_BF16: return launch_attn_tc<__nv_bfloat16>(mq, mk, mv, prm, split_p, s);
    default: return launch_attn_tc<__half>(mq, mk, mv, prm, split_p, s);
  }
}
}  // namespace h3s

extern "C" int h3s_sparse_attn_fwd(const int8_t *q8, const int8_t *k8, const uint8_t *v8t,
                                   const float *q_scale, const float *k_scale, const float *v_scale,
                                   const int32_t *route, int route_len, int q_start, int q_stop,
                                   void *out, int out_dtype, int64_t out_stride_h, int64_t out_stride_s,
                                   int heads, int sequence, int flags, int32_t *status,
                                   h3s_stream_t stream) {
  return h3s::sparse_attn_fwd_impl(q8, k8, v8t, q_scale, k_scale, v_scale, route, route_len, q_start, q_stop, out,
                                   nullptr, 0, out_dtype, out_stride_h, out_stride_s, heads, sequence, flags,
                                   status, stream);
}

extern "C" int h3s_sparse_attn_fwd_scatter(const int8_t *q8, const int8_t *k8, const uint8_t *v8t,
                                           const float *q_scale, const float *k_scale, const float *v_scale,
                                           const int32_t *route, int route_len, int q_start, int q_stop,
                                           void *out, void *const *peer_out, int n_peer_out, int out_dtype,
                                           int64_t out_stride_h, int64_t out_stride_s, int heads, int sequence,
                                           int flags, int32_t *status, h3s_stream_t stream) {
  return h3s::sparse_attn_fwd_impl(q8, k8, v8t, q_scale, k_scale, v_scale, route, route_len, q_start, q_stop, out,
                                   peer_out, n_peer_out, out_dtype, out_stride_h, out_stride_s, heads, sequence,
                                   flags, status, stream);
}
