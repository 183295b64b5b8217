/*
 * h3sparse.h - C ABI of the B200 (sm_100a) sparse-attention hot path.
 *
 * Every entry point takes raw device pointers, explicit strides/sizes and a
 * CUDA stream, launches asynchronously on that stream, never allocates, never
 * synchronises, and returns 0 on success or a negative H3S_E* code (message
 * in h3s_last_error(), thread-local).  Strides are in ELEMENTS of the tensor
 * they describe.  "HND" means a (heads, sequence, 128) view whose last
 * dimension is contiguous; batch is always 1 (reference:
 * attention/sparse/sparse_sage.py:448-449) - callers loop over batch.
 *
 * Each declaration cites the reference interface it replaces
 * (file:line inside Pizzawookiee/H3-Optimizations).
 */
#ifndef H3SPARSE_H_
#define H3SPARSE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define H3S_OK 0
#define H3S_EINVAL (-1)   /* bad argument (shape, alignment, dtype)          */
#define H3S_ECUDA (-2)    /* a CUDA runtime/driver call failed                */
#define H3S_EARCH (-3)    /* device is not sm_100                             */
#define H3S_ETIMEOUT (-4) /* a device-side bounded wait ran out (status word) */

#define H3S_Q_TILE 128
#define H3S_KV_TILE 64
#define H3S_HEAD_DIM 128

/* element types of floating inputs/outputs */
#define H3S_F32 0
#define H3S_BF16 1
#define H3S_F16 2
#define H3S_F64 3 /* router summaries only */

typedef void *h3s_stream_t; /* cudaStream_t */

/* Library / device ---------------------------------------------------- */

/* ABI version of this header (bumped on any signature change). */
int h3s_abi_version(void);
/* Message of the last failing call on this host thread ("" if none). */
const char *h3s_last_error(void);
/* Compute capability of the current device as major*10+minor (100 on B200);
 * replaces the capability gate of attention/sparse/sparse_sage.py:274-277. */
int h3s_device_capability(void);

/* Carrier quantisation -------------------------------------------------- */

/* Bytes of scratch h3s_column_stats needs for `heads` heads. */
size_t h3s_column_stats_scratch_bytes(int heads);

/*
 * Whole-sequence per-(head,channel) statistics, one pass over K and V:
 *   k_mean[h,d] = mean_s K[h,s,d]  rounded to `dtype` and widened to fp32
 *   v_scale[h,d] = max(max_s |V[h,s,d]| / v_bound, 1e-20)
 * Either of k / v may be NULL (its output is then untouched).
 * `scratch` (h3s_column_stats_scratch_bytes) is cleared by the call itself.
 * Replaces `k.mean(dim=-2)` (attention/sparse/sparse_sage.py:319,
 * sparse_quant.py:105) and update_v_amax / finalize_v_scale
 * (attention/sparse/fp8_v_stream.py:58-66).
 */
int h3s_column_stats(const void *k, int64_t k_stride_h, int64_t k_stride_s,
                     const void *v, int64_t v_stride_h, int64_t v_stride_s,
                     int dtype, int heads, int sequence, float v_bound,
                     float *k_mean, float *v_scale, void *scratch,
                     h3s_stream_t stream);

/*
 * h3s_column_stats for hosts that have no scratch buffer to give.  (No
 * counterpart in the reference: its statistics are torch reductions.)
 *
 * Some hosts of this library run under a closed memory plan: a serving
 * process that froze its device pool after warm-up, or a plug-in called from
 * inside another framework's operator where that framework's allocator must
 * not be re-entered.  They can still pass inputs and outputs they already
 * own, but not the extra `scratch` that h3s_column_stats asks for.  This
 * variant keeps that scratch inside the library instead (a 96 KiB array in
 * device memory, one copy on every GPU that loads the library, held until
 * the process exits), so the call allocates nothing, here or in any library.
 *
 * Same arguments, results and errors as h3s_column_stats minus `scratch`,
 * with these limits:
 *   - heads <= 64; more is rejected with H3S_EINVAL and a message naming
 *     the limit (use h3s_column_stats with your own scratch then);
 *   - the first call on each device looks up the array's device address
 *     (with that device current); make that first call outside any stream
 *     capture;
 *   - every call on a device shares the one array.  The call clears the part
 *     it uses before accumulating, so leftovers of an earlier call never leak
 *     into a result, but two calls that overlap on the GPU (different
 *     streams, no ordering between them) race on it and both results are
 *     then undefined.  Order them on one stream or with events.
 */
int h3s_column_stats_static(const void *k, int64_t k_stride_h,
                            int64_t k_stride_s, const void *v,
                            int64_t v_stride_h, int64_t v_stride_s, int dtype,
                            int heads, int sequence, float v_bound,
                            float *k_mean, float *v_scale,
                            h3s_stream_t stream);

/*
 * Per-block INT8 quantisation of an HND tensor (Q: block 128, K: block 64):
 *   v = x - mean[h,:] (mean may be NULL);  scale = amax|v|/127 + 1e-7;
 *   code = trunc(v/scale +- 0.5).
 * Rows [0,rows) of `x` are rows [row_start,row_start+rows) of the carrier;
 * row_start must be a multiple of `block`; only the last block may be ragged.
 * out:      int8  (heads, sequence_total, 128) contiguous
 * scale:    fp32  (heads, ceil(sequence_total/block))
 * summary:  optional tile means, element type `summary_dtype`
 *           (heads, blocks_total, 128); H3S_F64 stores the exact FP64 mean
 *           used by the router, other types store the FP32 mean rounded.
 * out and scale may both be NULL (pooling only: just the tile means).
 * Replaces _quantize_blocks (attention/sparse/sparse_sage.py:312-330,
 * sparse_quant.py:8-70) and pack_sparse_qk_chunk_into
 * (attention/sparse/chunked_qkv.py:33-191).
 */
int h3s_quant_qk_blocks(const void *x, int dtype, int64_t x_stride_h,
                        int64_t x_stride_s, const float *mean, int8_t *out,
                        float *scale, void *summary, int summary_dtype,
                        int heads, int rows, int row_start,
                        int sequence_total, int block, h3s_stream_t stream);

/*
 * FP8-E4M3 V carrier: out[h,d,row_start+s] = e4m3(clamp(V[h,s,d]/scale[h,d],
 * +-v_bound)); out is (heads, 128, pad128(sequence_total)) contiguous and the
 * padding columns of the final chunk are written as zero.
 * Replaces prepare_v / pack_v_chunk (attention/sparse/sparse_sage.py:84-110,
 * attention/sparse/fp8_v_stream.py:14-55,78-140).
 */
int h3s_quant_v_fp8(const void *v, int dtype, int64_t v_stride_h,
                    int64_t v_stride_s, const float *v_scale, uint8_t *out,
                    int heads, int rows, int row_start, int sequence_total,
                    float v_bound, h3s_stream_t stream);

/* Chunked QKV projection -------------------------------------------------- */

/*
 * ConvRot activation quantisation for one chunk of rows: every 256-channel
 * group of a row is rotated by the normalised Sylvester Hadamard matrix
 * H256/16 (fast Walsh-Hadamard transform in FP32, stages in ascending stride
 * order), then the row is quantised to INT8 with scale = amax/127 (1 when the
 * row is zero), code = rint(v/scale) clamped to +-127.
 *   x       bf16 (rows, hidden), row stride in elements, hidden % 256 == 0
 *   x_i8    int8 (rows, hidden) contiguous;  x_scale fp32 (rows)
 * Replaces comfy_kitchen quantize_int8_rowwise_convrot64(x, 256) as called at
 * attention/sparse/fused_qkv.py:489-496 (the rotation itself is defined by the
 * benchmark configuration; the reference does not vendor it).
 */
int h3s_convrot_quant_rows(const void *x, int64_t x_stride_row, int rows,
                           int hidden, int8_t *x_i8, float *x_scale,
                           h3s_stream_t stream);

/*
 * INT8 GEMM + de-quantisation for one chunk (tcgen05 kind::i8, TMA fed):
 *   y[row, n] = bf16( float(sum_k x_i8[row,k] * w_i8[n,k]) * (x_scale[row] * w_scale[n]) )
 * w_i8 int8 (n_out, hidden) contiguous, rows ordered [Q heads | K heads | V heads]
 * (row kind*H*128 + head*128 + d); n_out and hidden multiples of 128.
 * Output is head-major: 128-column group g (= kind*H + head) of row r lands at
 *   out_bf16 + g*out_stride_head + r*128,
 * so a (3*H, S, 128) staging tensor receives chunk rows [row_start, ...) when
 * the caller offsets out_bf16 by row_start*128 and passes out_stride_head = S*128.
 * status: optional device int32[4], word 0 non-zero if a bounded device wait
 * expired.
 * Replaces _fused_qk_kernel / _fused_v_kernel GEMM + dequant
 * (attention/sparse/fused_qkv.py:198-223,370-438) and project_chunk_hnd
 * (qkv/chunked.py:6-10).
 */
int h3s_qkv_gemm_chunk(const int8_t *x_i8, const float *x_scale,
                       const int8_t *w_i8, const float *w_scale, int rows,
                       int hidden, int n_out, void *out_bf16,
                       int64_t out_stride_head, int32_t *status,
                       h3s_stream_t stream);

/*
 * The same GEMM with the per-head RMS norm and the split-half rotary embedding
 * of the Q and K heads applied in its epilogue (V heads pass through):
 *   y    = bf16(acc * (x_scale[row] * w_scale[col]))
 *   y    = bf16(y * rsqrt(mean_d(y^2) + epsilon) * norm[d])       norm = q_norm | k_norm, fp32 (128)
 *   y[d], y[d+48] = bf16(f00*y[d] + f01*y[d+48]), bf16(f10*y[d] + f11*y[d+48])   for d < 48
 * with f(a,b) = rope[row*rope_strides[0] + d*rope_strides[1] + a*rope_strides[2]
 * + b*rope_strides[3]] (element strides; rope_dtype H3S_F32 or H3S_BF16), i.e.
 * the (1,S,1,48,2,2) tensor of the model offset to the chunk's first row.
 * rope == NULL: norm only.  n_out = 3*heads*128.
 * Replaces the norm/rotation part of _fused_qk_kernel
 * (attention/sparse/fused_qkv.py:225-289) and rms_rope_split_half_ as used in
 * attention_forward.py:10-48.
 */
int h3s_qkv_gemm_chunk_norm_rope(const int8_t *x_i8, const float *x_scale,
                                 const int8_t *w_i8, const float *w_scale,
                                 int rows, int hidden, int heads,
                                 void *out_bf16, int64_t out_stride_head,
                                 const float *q_norm, const float *k_norm,
                                 float epsilon, const void *rope,
                                 int rope_dtype, const int64_t *rope_strides,
                                 int32_t *status, h3s_stream_t stream);

/* Router ---------------------------------------------------------------- */

/*
 * Top-`retained` pure-video KV tiles for every pure-video query tile, from
 * tile means.  q_summary (heads,q_tiles,128), k_summary (heads,kv_tiles,128)
 * of element type `dtype` (H3S_F64/F32/BF16/F16), contiguous.
 * Pure-video tiles are [q_start,q_stop) and [kv_start,kv_stop).
 * route: int32 (heads, q_stop-q_start, route_len) with
 *   route_len = kv_tiles - (kv_stop-kv_start) + retained,
 * each row = ascending absolute KV tile indices: the non-video tiles plus the
 * selected ones.  Scores are exact FP64 dot products; equal scores keep the
 * lower tile index.
 * Replaces SparseTileRouter._build_lut_from_summaries / _pack_rows
 * (attention/sparse/router.py:38-56,453-531) and
 * build_compact_absolute_route (attention/sparse/triton_route.py:42-93).
 */
int h3s_route_topk(const void *q_summary, const void *k_summary, int dtype,
                   int heads, int q_tiles, int kv_tiles, int q_start,
                   int q_stop, int kv_start, int kv_stop, int retained,
                   int32_t *route, h3s_stream_t stream);

/*
 * Expand a compact route into the reference's delta-encoded LUT
 * lut int32 (heads,q_tiles,kv_tiles) and valid int32 (heads,q_tiles)
 * (attention/sparse/router.py:219-240,453-475).  route may be NULL (dense).
 */
int h3s_route_to_delta_lut(const int32_t *route, int heads, int q_tiles,
                           int kv_tiles, int q_start, int q_stop,
                           int route_len, int32_t *lut, int32_t *valid,
                           h3s_stream_t stream);

/*
 * Carrier outputs of h3s_qkv_gemm_chunk_carriers.  Every tensor covers the
 * WHOLE sequence of `sequence_total` rows (the chunk lands at row_start):
 *   q8, k8        int8 (heads, sequence_total, 128)
 *   q_scale       fp32 (heads, ceil(S/128));  k_scale fp32 (heads, ceil(S/64))
 *   q_summary     (heads, ceil(S/128), 128), k_summary (heads, ceil(S/64), 128):
 *                 tile means of the de-quantised (normed, rotated) Q and K,
 *                 element type summary_dtype
 *   k_stage, v_stage  bf16 (heads, sequence_total, 128)
 *   stats         h3s_column_stats_scratch_bytes(heads) bytes, zeroed by the
 *                 caller before the first chunk of a sequence
 * K is either quantised per chunk like Q (k8 + k_scale given, k_stage NULL: no
 * mean smoothing, what the reference's chunked producers do,
 * attention/sparse/chunked_qkv.py:289) or staged in bf16 (k_stage given, k8 and
 * k_scale NULL) while its column sums accumulate in `stats`, to be quantised
 * with the whole-sequence mean removed once every chunk is through.  V is
 * always staged while its column maxima accumulate in `stats`.
 */
typedef struct h3s_qkv_carriers {
  int8_t *q8;
  float *q_scale;
  void *q_summary;
  int8_t *k8;
  float *k_scale;
  void *k_summary;
  void *k_stage;
  void *v_stage;
  void *stats;
  int summary_dtype;
  int sequence_total;
  int row_start;
} h3s_qkv_carriers;

/*
 * h3s_qkv_gemm_chunk[_norm_rope] whose epilogue emits carriers instead of bf16
 * staging: per 128-row Q block of a head the block amax, scale = amax/127+1e-7,
 * INT8 codes trunc(y/scale +- 0.5) and the tile mean; the same per 64-row K
 * block when K is not smoothed (see h3s_qkv_carriers).  q_norm/k_norm/rope as
 * in h3s_qkv_gemm_chunk_norm_rope, all three may be NULL.  rows must be a
 * multiple of 128 except in the final chunk of the sequence.
 * Replaces _fused_qk_kernel / _fused_v_kernel including their quantising
 * epilogues (attention/sparse/fused_qkv.py:292-367,427-438) and the per-chunk
 * packing of pack_sparse_qk_chunk_into (attention/sparse/chunked_qkv.py:119-203,247-273).
 */
int h3s_qkv_gemm_chunk_carriers(const int8_t *x_i8, const float *x_scale,
                                const int8_t *w_i8, const float *w_scale,
                                int rows, int hidden, int heads,
                                const h3s_qkv_carriers *carriers,
                                const float *q_norm, const float *k_norm,
                                float epsilon, const void *rope, int rope_dtype,
                                const int64_t *rope_strides, int32_t *status,
                                h3s_stream_t stream);

/*
 * Second phase of the statistics that h3s_qkv_gemm_chunk_carriers accumulates
 * (or any scratch in h3s_column_stats' layout): k_mean = sum/sequence rounded to
 * `dtype` and widened, v_scale = max(amax/v_bound, 1e-20); either output may be
 * NULL.  Replaces finalize_v_scale (attention/sparse/fp8_v_stream.py:58-66) and
 * the mean of attention/sparse/sparse_sage.py:319.
 */
int h3s_column_stats_finalize(const void *stats, int dtype, int heads,
                              int sequence, float v_bound, float *k_mean,
                              float *v_scale, h3s_stream_t stream);

/* Dense GEMM --------------------------------------------------------------- */

#define H3S_GEMM_I8 0    /* int8 x int8, int32 accumulation   */
#define H3S_GEMM_BF16 1  /* bf16 x bf16, fp32 accumulation    */
#define H3S_GEMM_F16 2   /* fp16 x fp16, fp32 accumulation    */
#define H3S_GEMM_E4M3 3  /* e4m3 x e4m3, fp32 accumulation    */
#define H3S_ACT_NONE 0
#define H3S_ACT_GELU_TANH 1

/*
 * out[m, n] = bf16( act( (sum_k a[m,k] * b[n,k]) * row_scale[m] * col_scale[n] + bias[n] ) )
 * on the tcgen05 tensor cores (the persistent TMA-fed kernel of the QKV
 * projection with a row-major epilogue whose stores are staged through shared
 * memory and leave as full lines).
 *   a        (rows, K) elements of `operand_kind`, row stride lda_bytes
 *   b        (n_out, K), row stride ldb_bytes: a torch Linear weight as stored
 *   k_bytes  K * element size, a multiple of 128
 *   row_scale (rows), col_scale (n_out), bias (n_out): fp32, each may be NULL
 *   activation H3S_ACT_NONE or H3S_ACT_GELU_TANH (torch's approximate='tanh')
 *   out_bf16 (rows, ldc) bf16, n_out a multiple of 8
 * Replaces the attention module's out_proj call behind execute_projected
 * (attention_forward.py:99-128, attention/sparse/sparse_sage_streamed.py:1454-1472)
 * and the two FP8 linears of the chunked MLP (memory/linear.py:352-492,
 * memory/forward.py:138-298).
 */
int h3s_dense_gemm(const void *a, int64_t lda_bytes, const void *b,
                   int64_t ldb_bytes, int operand_kind, int rows, int n_out,
                   int k_bytes, const float *row_scale, const float *col_scale,
                   const float *bias, int activation, void *out_bf16,
                   int64_t ldc, int32_t *status, h3s_stream_t stream);

/*
 * Per-row FP8-E4M3 quantisation of a bf16 matrix: scale[m] = max(amax_m / 448,
 * 1e-20), code = e4m3(x / scale[m]).  x (rows, channels) with row stride in
 * elements, channels a multiple of 8; out (rows, channels) contiguous.
 * Replaces the activation quantisation in front of the FP8 linears
 * (memory/linear.py:352-492).
 */
int h3s_quant_rows_fp8(const void *x_bf16, int64_t x_stride_row, int rows,
                       int channels, uint8_t *out, float *row_scale,
                       h3s_stream_t stream);

/*
 * Upper bound, in nanoseconds, of every wait inside the tcgen05 kernels
 * (attention and QKV GEMM) launched after the call; default 2 s, accepted range
 * 1 us .. 60 s.  A wait that runs out ends the kernel with a code in the
 * launch's status words (attention: 1 Q tile load, 2 K/V tile load, 3 free
 * K/V stage, 4 QK^T result, 5 P from the softmax warps, 6 free P buffer,
 * 7 P.V before a rescale, 8 last P.V; GEMM: 21 operand stage, 22 free stage,
 * 23 accumulator, 24 free accumulator), followed by the CTA index and, for
 * attention, the head and the query tile.  Process-wide.  No counterpart in
 * the reference (its Triton kernels have no device-side waits).
 */
int h3s_set_wait_budget_ns(unsigned long long nanoseconds);
unsigned long long h3s_get_wait_budget_ns(void);

/* Attention ------------------------------------------------------------- */

#define H3S_ATTN_P_SINGLE 1
/* Self-test of the bounded device waits: the K/V load of the first iteration is
 * never issued, so the wait for it gives up after the wait budget, the kernel
 * writes its status words, releases its tensor memory and returns.  The output
 * of such a launch is meaningless.  Nothing faults and nothing hangs. */
#define H3S_ATTN_TEST_DROP_KV_LOAD 0x4000
#define H3S_MAX_PEER_OUTPUTS 7

/*
 * Block-sparse attention on the carriers (tcgen05 kind::i8 QK^T into TMEM,
 * FP32 online softmax, kind::f8f6f4 P.V, TMA loads of the listed KV tiles).
 *   q8,k8   int8 (heads, sequence, 128) contiguous
 *   v8t     e4m3 (heads, 128, pad128(sequence)) contiguous, zero padded
 *   q_scale (heads, ceil(S/128)), k_scale (heads, ceil(S/64)), v_scale (heads,128)
 *   route   int32 (heads, q_stop-q_start, route_len) or NULL for fully dense;
 *           query tiles outside [q_start,q_stop) attend every KV tile.
 *   out     element type out_dtype (BF16/F16/F32), strides in elements.
 *   flags   0, or H3S_ATTN_P_SINGLE to carry P as one E4M3 term instead of
 *           two (hi + lo): fewer MMAs, ~2.5e-2 instead of ~2e-3 relative error.
 *   status  device int32[4]; word 0 is set non-zero if a bounded device wait
 *           expired (the output is then invalid); may be NULL.
 * Replaces the kernel call of attention/sparse/sparse_sage.py:112-121 and
 * launch_int8_sparse (attention/sparse/triton_sparse_kernels.py:206-246).
 */
int h3s_sparse_attn_fwd(const int8_t *q8, const int8_t *k8, const uint8_t *v8t,
                        const float *q_scale, const float *k_scale,
                        const float *v_scale, const int32_t *route,
                        int route_len, int q_start, int q_stop, void *out,
                        int out_dtype, int64_t out_stride_h,
                        int64_t out_stride_s, int heads, int sequence,
                        int flags, int32_t *status, h3s_stream_t stream);

/*
 * h3s_sparse_attn_fwd for head-sharded runs (one process per GPU, this rank
 * holds `heads` of the layer's heads): besides `out`, every output tile is
 * stored with plain peer-to-peer stores into `n_peer_out` (<= 7) further
 * buffers - the slice of each peer GPU's full (H_total,S,128) output that
 * belongs to this rank's heads, mapped into this process (e.g. CUDA IPC or
 * torch symmetric memory) and addressed with the same strides as `out`.  The
 * attention kernel thereby performs the all-gather of the head-sharded output
 * itself, tile by tile over NVLink; the caller only needs a cross-rank barrier
 * before a peer reads its buffer.  No TMA, no multicast touches peer memory.
 * (No counterpart in the reference, which is single-GPU.)
 */
int h3s_sparse_attn_fwd_scatter(const int8_t *q8, const int8_t *k8,
                                const uint8_t *v8t, const float *q_scale,
                                const float *k_scale, const float *v_scale,
                                const int32_t *route, int route_len,
                                int q_start, int q_stop, void *out,
                                void *const *peer_out, int n_peer_out,
                                int out_dtype, int64_t out_stride_h,
                                int64_t out_stride_s, int heads, int sequence,
                                int flags, int32_t *status,
                                h3s_stream_t stream);

/*
 * Same contract, legacy tensor path (mma.sync m16n8k32 s8 / e4m3).  Kept as
 * the on-device cross-check of the tcgen05 kernel; not used by the backend.
 */
int h3s_sparse_attn_fwd_mma(const int8_t *q8, const int8_t *k8,
                            const uint8_t *v8t, const float *q_scale,
                            const float *k_scale, const float *v_scale,
                            const int32_t *route, int route_len, int q_start,
                            int q_stop, void *out, int out_dtype,
                            int64_t out_stride_h, int64_t out_stride_s,
                            int heads, int sequence, int flags,
                            h3s_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* H3SPARSE_H_ */
