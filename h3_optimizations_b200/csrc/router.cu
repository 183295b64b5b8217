// Block router: exact FP64 tile-mean scores, per-row radix top-k, ordered
// emission of the packed KV-tile index list.
//
// One CTA scores 8 pure-video query tiles of one head against every
// pure-video KV tile with FP64 tensor-core MMAs (scores kept in shared
// memory).  The K tile means are brought in 64 tiles at a time by the whole
// CTA with coalesced loads (every thread has 32 independent loads in flight)
// and widened to FP64 in shared memory; the MMA operands are then read from
// there.  Each warp then owns one row: an 8-pass MSB-first radix select on
// order-preserving 64-bit keys finds the retained-th largest score exactly,
// and a ballot-ordered sweep writes the surviving tile indices in ascending
// order, so no sort is needed.
#include "common.cuh"

namespace h3s {

constexpr int kRouteRows = 8;         // query tiles per CTA == warps per CTA
constexpr int kRouteThreads = kRouteRows * 32;
constexpr int kRouteKBlock = 64;       // KV tiles staged per round: one 8-tile MMA block per warp
// Row stride of the staged block in doubles: 128 channels + 4 of padding, so the
// 16 lanes of a half warp (4 tiles x 4 channels) read 16 different 8-byte banks.
constexpr int kRouteKStride = H3S_HEAD_DIM + 4;

template <typename T> __device__ __forceinline__ double to_double(T v);
template <> __device__ __forceinline__ double to_double<double>(double v) { return v; }
template <> __device__ __forceinline__ double to_double<float>(float v) { return static_cast<double>(v); }
template <> __device__ __forceinline__ double to_double<__nv_bfloat16>(__nv_bfloat16 v) { return static_cast<double>(__bfloat162float(v)); }
template <> __device__ __forceinline__ double to_double<__half>(__half v) { return static_cast<double>(__half2float(v)); }

// larger score <=> larger key
__device__ __forceinline__ unsigned long long score_key(double s) {
  const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(s));
  return (bits >> 63) ? ~bits : (bits | 0x8000000000000000ull);
}

template <typename T>
__global__ void __launch_bounds__(kRouteThreads)
route_topk_kernel(const T *__restrict__ q_summary, const T *__restrict__ k_summary, int q_tiles,
                  int kv_tiles, int q_start, int q_stop, int kv_start, int kv_stop, int retained,
                  int route_len, int32_t *__restrict__ route) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int pure_q = q_stop - q_start;
  const int pure_kv = kv_stop - kv_start;
  double *scores = reinterpret_cast<double *>(smem_raw);                                     // [kRouteRows][pure_kv]
  double *k_block = scores + static_cast<size_t>(kRouteRows) * pure_kv;                     // [kRouteKBlock][kRouteKStride]
  int *hist = reinterpret_cast<int *>(k_block + kRouteKBlock * kRouteKStride);              // [rows][256]

  const int head = blockIdx.y;
  const int row0 = blockIdx.x * kRouteRows;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- scores[r][p] = <q[r], k[p]> in FP64 on the tensor cores ----
  // mma.m8n8k4.f64: A is the CTA's 8 query tiles x 4 channels, B 4 channels x 8
  // KV tiles; lane l holds A[l/4][l%4], B[l%4][l/4] and C[l/4][2*(l%4) + {0,1}].
  // The 32 A fragments of a lane (all 128 channels) stay in registers.
  {
    const int frag_row = lane >> 2, frag_k = lane & 3;
    const int a_row = min(row0 + frag_row, pure_q - 1);
    const T *qp = q_summary + (static_cast<int64_t>(head) * q_tiles + q_start + a_row) * H3S_HEAD_DIM + frag_k;
    double a[H3S_HEAD_DIM / 4];
#pragma unroll
    for (int kk = 0; kk < H3S_HEAD_DIM / 4; ++kk) a[kk] = to_double(qp[4 * kk]);
    const T *k_head = k_summary + (static_cast<int64_t>(head) * kv_tiles + kv_start) * H3S_HEAD_DIM;
    for (int base = 0; base < pure_kv; base += kRouteKBlock) {
      // stage tiles [base, base + 64): element e of the block is channel e % 128 of tile e / 128
      constexpr int kPerThread = kRouteKBlock * H3S_HEAD_DIM / kRouteThreads;  // 32
      T staged[kPerThread];
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) {
        const int e = i * kRouteThreads + threadIdx.x;
        const int tile = min(base + (e >> 7), pure_kv - 1);  // rows past the end repeat the last tile
        staged[i] = k_head[static_cast<int64_t>(tile) * H3S_HEAD_DIM + (e & 127)];
      }
      __syncthreads();  // the previous round's readers are done with k_block
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) {
        const int e = i * kRouteThreads + threadIdx.x;
        k_block[(e >> 7) * kRouteKStride + (e & 127)] = to_double(staged[i]);
      }
      __syncthreads();
      const double *kp = k_block + (8 * warp + frag_row) * kRouteKStride + frag_k;
      double c0 = 0.0, c1 = 0.0;
#pragma unroll
      for (int kk = 0; kk < H3S_HEAD_DIM / 4; ++kk) {
        const double b = kp[4 * kk];
        asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                     : "+d"(c0), "+d"(c1)
                     : "d"(a[kk]), "d"(b));
      }
      const int col = base + 8 * warp + 2 * frag_k;
      if (col < pure_kv) scores[static_cast<size_t>(frag_row) * pure_kv + col] = c0;
      if (col + 1 < pure_kv) scores[static_cast<size_t>(frag_row) * pure_kv + col + 1] = c1;
    }
  }
  __syncthreads();

  // ---- per-warp exact selection ----
  const int row = row0 + warp;
  if (row >= pure_q) return;
  const double *srow = scores + static_cast<size_t>(warp) * pure_kv;
  int *h = hist + warp * 256;

  unsigned long long prefix = 0ull, prefix_mask = 0ull;
  int k_rem = retained;
  for (int shift = 56; shift >= 0; shift -= 8) {
    for (int b = lane; b < 256; b += 32) h[b] = 0;
    __syncwarp();
    for (int i = lane; i < pure_kv; i += 32) {
      const unsigned long long key = score_key(srow[i]);
      if ((key & prefix_mask) == prefix) atomicAdd(&h[(key >> shift) & 0xff], 1);
    }
    __syncwarp();
    // lane L owns bins 255-8L .. 248-8L (descending); find where the running
    // count from the top first reaches k_rem
    int mine[8];
    int sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { mine[j] = h[255 - (lane * 8 + j)]; sum += mine[j]; }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    const int excl = incl - sum;
    const bool owner = excl < k_rem && k_rem <= incl;
    int digit = 0, above = 0;
    if (owner) {
      int run = excl;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (run < k_rem && k_rem <= run + mine[j]) { digit = 255 - (lane * 8 + j); above = run; }
        run += mine[j];
      }
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, owner);
    const int src = __ffs(ballot) - 1;  // exactly one owner because sum(h) >= k_rem
    digit = __shfl_sync(0xffffffffu, digit, src);
    above = __shfl_sync(0xffffffffu, above, src);
    k_rem -= above;
    prefix |= static_cast<unsigned long long>(digit) << shift;
    prefix_mask |= 0xffull << shift;
    __syncwarp();
  }
  const unsigned long long threshold = prefix;  // retained-th largest key; take k_rem of its ties

  // ---- ordered emission: context before, selected ascending, context after ----
  int32_t *dst = route + (static_cast<int64_t>(head) * pure_q + row) * route_len;
  for (int i = lane; i < kv_start; i += 32) dst[i] = i;
  int base = kv_start;
  int ties_seen = 0;
  const unsigned lt_mask = (1u << lane) - 1u;
  for (int i0 = 0; i0 < pure_kv; i0 += 32) {
    const int i = i0 + lane;
    unsigned long long key = 0ull;
    const bool in = i < pure_kv;
    if (in) key = score_key(srow[i]);
    const bool eq = in && key == threshold;
    const unsigned eq_mask = __ballot_sync(0xffffffffu, eq);
    const bool take = in && (key > threshold || (eq && ties_seen + __popc(eq_mask & lt_mask) < k_rem));
    const unsigned take_mask = __ballot_sync(0xffffffffu, take);
    if (take) dst[base + __popc(take_mask & lt_mask)] = kv_start + i;
    base += __popc(take_mask);
    ties_seen += __popc(eq_mask);
  }
  for (int i = kv_stop + lane; i < kv_tiles; i += 32) dst[base + (i - kv_stop)] = i;
}

__global__ void route_to_delta_lut_kernel(const int32_t *__restrict__ route, int q_tiles, int kv_tiles,
                                          int q_start, int q_stop, int route_len,
                                          int32_t *__restrict__ lut, int32_t *__restrict__ valid) {
  const int tq = blockIdx.x, head = blockIdx.y;
  int32_t *row = lut + (static_cast<int64_t>(head) * q_tiles + tq) * kv_tiles;
  const bool sparse = route != nullptr && tq >= q_start && tq < q_stop;
  const int32_t *src = sparse ? route + (static_cast<int64_t>(head) * (q_stop - q_start) + (tq - q_start)) * route_len : nullptr;
  for (int j = threadIdx.x; j < kv_tiles; j += blockDim.x) {
    int32_t value = j == 0 ? 0 : 1;
    if (sparse && j < route_len) value = src[j] - (j ? src[j - 1] : 0);
    row[j] = value;
  }
  if (threadIdx.x == 0) valid[head * q_tiles + tq] = sparse ? route_len : kv_tiles;
}

template <typename T>
static int launch_route(const void *q_summary, const void *k_summary, int heads, int q_tiles, int kv_tiles,
                        int q_start, int q_stop, int kv_start, int kv_stop, int retained, int route_len,
                        int32_t *route, cudaStream_t stream) {
  const int pure_q = q_stop - q_start, pure_kv = kv_stop - kv_start;
  const size_t smem = sizeof(double) * (static_cast<size_t>(kRouteRows) * pure_kv + kRouteKBlock * kRouteKStride) +
                      sizeof(int) * kRouteRows * 256;
  H3S_CHECK_ARG(smem <= 220 * 1024, "route_topk: %d pure-video KV tiles need %zu bytes of shared memory", pure_kv, smem);
  H3S_CHECK_CUDA(cudaFuncSetAttribute(route_topk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  dim3 grid(ceil_div(pure_q, kRouteRows), heads);
  route_topk_kernel<T><<<grid, kRouteThreads, smem, stream>>>(
      static_cast<const T *>(q_summary), static_cast<const T *>(k_summary), q_tiles, kv_tiles, q_start,
      q_stop, kv_start, kv_stop, retained, route_len, route);
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

}  // namespace h3s

extern "C" {

int h3s_route_topk(const void *q_summary, const void *k_summary, int dtype, int heads, int q_tiles,
                   int kv_tiles, int q_start, int q_stop, int kv_start, int kv_stop, int retained,
                   int32_t *route, h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(q_summary != nullptr && k_summary != nullptr && route != nullptr, "route_topk: NULL pointer");
  H3S_CHECK_ARG(heads > 0 && q_tiles > 0 && kv_tiles > 0, "route_topk: empty problem");
  H3S_CHECK_ARG(0 <= q_start && q_start < q_stop && q_stop <= q_tiles, "route_topk: bad query tile range [%d,%d) of %d", q_start, q_stop, q_tiles);
  H3S_CHECK_ARG(0 <= kv_start && kv_start < kv_stop && kv_stop <= kv_tiles, "route_topk: bad KV tile range [%d,%d) of %d", kv_start, kv_stop, kv_tiles);
  H3S_CHECK_ARG(retained >= 1 && retained <= kv_stop - kv_start, "route_topk: retained %d outside [1,%d]", retained, kv_stop - kv_start);
  const int route_len = kv_tiles - (kv_stop - kv_start) + retained;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case H3S_F64: return launch_route<double>(q_summary, k_summary, heads, q_tiles, kv_tiles, q_start, q_stop, kv_start, kv_stop, retained, route_len, route, s);
    case H3S_F32: return launch_route<float>(q_summary, k_summary, heads, q_tiles, kv_tiles, q_start, q_stop, kv_start, kv_stop, retained, route_len, route, s);
    case H3S_BF16: return launch_route<__nv_bfloat16>(q_summary, k_summary, heads, q_tiles, kv_tiles, q_start, q_stop, kv_start, kv_stop, retained, route_len, route, s);
    case H3S_F16: return launch_route<__half>(q_summary, k_summary, heads, q_tiles, kv_tiles, q_start, q_stop, kv_start, kv_stop, retained, route_len, route, s);
    default: return fail(H3S_EINVAL, "route_topk: unsupported summary dtype %d", dtype);
  }
}

int h3s_route_to_delta_lut(const int32_t *route, int heads, int q_tiles, int kv_tiles, int q_start,
                           int q_stop, int route_len, int32_t *lut, int32_t *valid,
                           h3s_stream_t stream) {
  using namespace h3s;
  H3S_CHECK_ARG(lut != nullptr && valid != nullptr, "route_to_delta_lut: NULL output");
  H3S_CHECK_ARG(heads > 0 && q_tiles > 0 && kv_tiles > 0, "route_to_delta_lut: empty problem");
  H3S_CHECK_ARG(route == nullptr || (0 <= q_start && q_start < q_stop && q_stop <= q_tiles && route_len > 0 && route_len <= kv_tiles),
                "route_to_delta_lut: bad route geometry");
  route_to_delta_lut_kernel<<<dim3(q_tiles, heads), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      route, q_tiles, kv_tiles, q_start, q_stop, route_len, lut, valid);
  H3S_CHECK_CUDA(cudaGetLastError());
  return H3S_OK;
}

}  // extern "C"
