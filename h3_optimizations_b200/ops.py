"""Tensor-level wrappers over the C ABI (one function per entry point).

All tensors must be CUDA tensors on the current device; every call launches on
torch's current stream and returns without synchronising.  Shapes follow the
reference's carriers: HND ``(1, H, S, 128)`` views with a contiguous last
dimension, scales ``(1, H, blocks)``, V carrier ``(1, H, 128, pad128(S))``.
"""

from __future__ import annotations

import ctypes

import torch

from . import _native
from ._native import check, dtype_code, ptr, stream_ptr

Q_TILE = 128
KV_TILE = 64
HEAD_DIM = 128
FP8_V_BOUND = 448.0
ATTN_P_SINGLE = 1
ATTN_TEST_DROP_KV_LOAD = 0x4000


def _ceil_div(a, b):
    return (a + b - 1) // b


def _hnd(x, what):
    if x.ndim != 4 or x.shape[0] != 1 or x.shape[-1] != HEAD_DIM or x.stride(-1) != 1:
        raise _native.NativeError("%s must be a (1,H,S,128) view with a contiguous last dimension" % what)
    if not x.is_cuda:
        raise _native.NativeError("%s must be a CUDA tensor (there is no CPU path)" % what)
    return x.shape[1], x.shape[2]


def device_capability():
    code = _native.load().h3s_device_capability()
    if code < 0:
        check(code, "h3s_device_capability")
    return code


def set_wait_budget_ns(nanoseconds):
    """Bound of every device-side wait of the kernels launched from now on
    (default 2 s).  Returns the previous value."""
    lib = _native.load()
    previous = int(lib.h3s_get_wait_budget_ns())
    check(lib.h3s_set_wait_budget_ns(int(nanoseconds)), "h3s_set_wait_budget_ns")
    return previous


def column_stats_buffers(heads, device, want_k_mean=True, want_v_scale=True):
    """``(k_mean | None, v_scale | None, scratch)`` for ``column_stats_into``."""
    lib = _native.load()
    scratch = torch.empty(lib.h3s_column_stats_scratch_bytes(int(heads)), dtype=torch.uint8, device=device)
    k_mean = torch.empty((1, heads, HEAD_DIM), dtype=torch.float32, device=device) if want_k_mean else None
    v_scale = torch.empty((1, heads, HEAD_DIM), dtype=torch.float32, device=device) if want_v_scale else None
    return k_mean, v_scale, scratch


def column_stats(k=None, v=None, v_bound=FP8_V_BOUND):
    """``(k_mean (1,H,128) | None, v_scale (1,H,128) | None)``."""
    ref = k if k is not None else v
    heads, _ = _hnd(ref, "column_stats input")
    k_mean, v_scale, scratch = column_stats_buffers(heads, ref.device, k is not None, v is not None)
    return column_stats_into(k, v, k_mean, v_scale, scratch, v_bound)


def column_stats_into(k, v, k_mean, v_scale, scratch, v_bound=FP8_V_BOUND):
    """``column_stats`` into caller-owned outputs and scratch (all from
    ``column_stats_buffers``), so that the launch can go to a stream other than
    the one the buffers were allocated on."""
    lib = _native.load()
    ref = k if k is not None else v
    heads, sequence = _hnd(ref, "column_stats input")
    if k is not None and v is not None and (k.shape != v.shape or k.dtype != v.dtype):
        raise _native.NativeError("column_stats: K and V must share shape and dtype")
    if (k is not None and k_mean is None) or (v is not None and v_scale is None):
        raise _native.NativeError("column_stats: an output buffer is missing")
    check(
        lib.h3s_column_stats(
            ptr(k), k.stride(1) if k is not None else 0, k.stride(2) if k is not None else 0,
            ptr(v), v.stride(1) if v is not None else 0, v.stride(2) if v is not None else 0,
            dtype_code(ref.dtype), heads, sequence, float(v_bound), ptr(k_mean), ptr(v_scale), ptr(scratch),
            stream_ptr(ref.device),
        ),
        "h3s_column_stats",
    )
    return k_mean, v_scale


def column_stats_static_into(k, v, k_mean, v_scale, v_bound=FP8_V_BOUND):
    """``column_stats`` into caller-owned ``k_mean`` / ``v_scale`` (fp32
    ``(1,H,128)``) with the scratch that is built into the library, so nothing
    is allocated by the call (at most 64 heads; calls that overlap on the GPU
    race on the shared scratch)."""
    lib = _native.load()
    ref = k if k is not None else v
    heads, sequence = _hnd(ref, "column_stats_static input")
    if k is not None and v is not None and (k.shape != v.shape or k.dtype != v.dtype):
        raise _native.NativeError("column_stats_static: K and V must share shape and dtype")
    for name, t, src in (("k_mean", k_mean, k), ("v_scale", v_scale, v)):
        if src is not None and (t is None or tuple(t.shape) != (1, heads, HEAD_DIM) or t.dtype != torch.float32
                                or not t.is_contiguous() or t.device != ref.device):
            raise _native.NativeError("column_stats_static: %s must be contiguous fp32 (1,H,128) on the input's device" % name)
    check(
        lib.h3s_column_stats_static(
            ptr(k), k.stride(1) if k is not None else 0, k.stride(2) if k is not None else 0,
            ptr(v), v.stride(1) if v is not None else 0, v.stride(2) if v is not None else 0,
            dtype_code(ref.dtype), heads, sequence, float(v_bound), ptr(k_mean), ptr(v_scale),
            stream_ptr(ref.device),
        ),
        "h3s_column_stats_static",
    )
    return k_mean, v_scale


def quant_qk_blocks_into(x, out, scale, summary, *, block, row_start=0, mean=None):
    """Quantise chunk ``x`` (1,H,rows,128) into rows ``[row_start, ...)`` of
    ``out`` (1,H,S_total,128) int8; ``scale`` (1,H,blocks_total);
    ``summary`` (1,H,blocks_total,128) or None.  ``out``/``scale`` may be None
    (pooling only)."""
    lib = _native.load()
    heads, rows = _hnd(x, "quant_qk_blocks input")
    if out is not None:
        sequence_total = out.shape[2]
        if out.dtype != torch.int8 or not out.is_contiguous() or out.shape[1] != heads:
            raise _native.NativeError("quant_qk_blocks: carrier must be contiguous int8 (1,H,S,128)")
        blocks_total = _ceil_div(sequence_total, block)
        if scale is None or tuple(scale.shape) != (1, heads, blocks_total) or scale.dtype != torch.float32 or not scale.is_contiguous():
            raise _native.NativeError("quant_qk_blocks: scale must be contiguous fp32 (1,H,%d)" % blocks_total)
    else:
        if summary is None:
            raise _native.NativeError("quant_qk_blocks: nothing to produce")
        sequence_total = None
    if summary is not None:
        blocks_total = summary.shape[2]
        if sequence_total is None:
            sequence_total = row_start + rows
        if (tuple(summary.shape) != (1, heads, _ceil_div(sequence_total, block), HEAD_DIM)
                or not summary.is_contiguous()):
            raise _native.NativeError("quant_qk_blocks: summary must be contiguous (1,H,blocks,128)")
    if mean is not None and (tuple(mean.shape) != (1, heads, HEAD_DIM) or mean.dtype != torch.float32 or not mean.is_contiguous()):
        raise _native.NativeError("quant_qk_blocks: mean must be contiguous fp32 (1,H,128)")
    check(
        lib.h3s_quant_qk_blocks(
            ptr(x), dtype_code(x.dtype), x.stride(1), x.stride(2), ptr(mean), ptr(out), ptr(scale),
            ptr(summary), dtype_code(summary.dtype) if summary is not None else 0, heads, rows,
            int(row_start), int(sequence_total), int(block), stream_ptr(x.device),
        ),
        "h3s_quant_qk_blocks",
    )


def quant_qk_blocks(x, block, *, mean=None, summary_dtype=None):
    """``(codes int8 (1,H,S,128), scale (1,H,blocks), summary | None)``."""
    heads, sequence = _hnd(x, "quant_qk_blocks input")
    blocks = _ceil_div(sequence, block)
    out = torch.empty((1, heads, sequence, HEAD_DIM), dtype=torch.int8, device=x.device)
    scale = torch.empty((1, heads, blocks), dtype=torch.float32, device=x.device)
    summary = None
    if summary_dtype is not None:
        summary = torch.empty((1, heads, blocks, HEAD_DIM), dtype=summary_dtype, device=x.device)
    quant_qk_blocks_into(x, out, scale, summary, block=block, mean=mean)
    return out, scale, summary


def tile_means(x, block, dtype=torch.float64):
    """Tile means only (no quantisation): ``(1,H,blocks,128)``."""
    heads, sequence = _hnd(x, "tile_means input")
    summary = torch.empty((1, heads, _ceil_div(sequence, block), HEAD_DIM), dtype=dtype, device=x.device)
    quant_qk_blocks_into(x, None, None, summary, block=block)
    return summary


def allocate_v_carrier(sequence, heads, device):
    """Zero-padded FP8 carrier ``(1,H,128,pad128(S))`` (reference:
    attention/sparse/fp8_v_stream.py:69-75).  Not cleared: the quantiser
    writes the padding itself."""
    padded = _ceil_div(int(sequence), 128) * 128
    return torch.empty((1, int(heads), HEAD_DIM, padded), dtype=torch.float8_e4m3fn, device=device)


def quant_v_fp8_into(v, v_scale, carrier, *, row_start=0, sequence_total=None, v_bound=FP8_V_BOUND):
    lib = _native.load()
    heads, rows = _hnd(v, "quant_v_fp8 input")
    sequence_total = int(sequence_total if sequence_total is not None else row_start + rows)
    padded = _ceil_div(sequence_total, 128) * 128
    if (tuple(carrier.shape) != (1, heads, HEAD_DIM, padded) or carrier.dtype != torch.float8_e4m3fn
            or not carrier.is_contiguous()):
        raise _native.NativeError("quant_v_fp8: carrier must be contiguous e4m3 (1,H,128,%d)" % padded)
    if tuple(v_scale.shape) != (1, heads, HEAD_DIM) or v_scale.dtype != torch.float32 or not v_scale.is_contiguous():
        raise _native.NativeError("quant_v_fp8: scale must be contiguous fp32 (1,H,128)")
    check(
        lib.h3s_quant_v_fp8(
            ptr(v), dtype_code(v.dtype), v.stride(1), v.stride(2), ptr(v_scale), ptr(carrier), heads, rows,
            int(row_start), sequence_total, float(v_bound), stream_ptr(v.device),
        ),
        "h3s_quant_v_fp8",
    )


def quant_v_fp8(v, v_scale=None, v_bound=FP8_V_BOUND):
    """``(carrier e4m3 (1,H,128,pad128(S)), scale (1,H,128))``."""
    heads, sequence = _hnd(v, "quant_v_fp8 input")
    if v_scale is None:
        _, v_scale = column_stats(None, v, v_bound)
    carrier = allocate_v_carrier(sequence, heads, v.device)
    quant_v_fp8_into(v, v_scale, carrier, v_bound=v_bound)
    return carrier, v_scale


def convrot_quant_rows(x, x_i8=None, x_scale=None):
    """ConvRot (Hadamard-256) + per-row INT8 of ``x`` (rows, hidden) bf16.
    Returns ``(codes int8 (rows, hidden), scale fp32 (rows,))``."""
    lib = _native.load()
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_cuda or x.stride(1) != 1:
        raise _native.NativeError("convrot_quant_rows: x must be a rank-2 CUDA bf16 tensor with contiguous rows")
    rows, hidden = x.shape
    if x_i8 is None:
        x_i8 = torch.empty((rows, hidden), dtype=torch.int8, device=x.device)
    if x_scale is None:
        x_scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
    if x_i8.shape[0] < rows or x_i8.shape[1] != hidden or not x_i8.is_contiguous() or x_scale.numel() < rows:
        raise _native.NativeError("convrot_quant_rows: output buffers are too small")
    check(
        lib.h3s_convrot_quant_rows(ptr(x), x.stride(0), rows, hidden, ptr(x_i8), ptr(x_scale), stream_ptr(x.device)),
        "h3s_convrot_quant_rows",
    )
    return x_i8[:rows], x_scale[:rows]


def qkv_gemm_chunk(x_i8, x_scale, w_i8, w_scale, staging, *, row_start=0, status=None,
                   q_norm=None, k_norm=None, epsilon=1e-6, rope=None):
    """INT8 GEMM of one chunk into ``staging`` bf16 ``(groups, S, 128)`` (group =
    kind*H + head) at rows ``[row_start, row_start + rows)``.

    With ``q_norm`` / ``k_norm`` (fp32 ``(128,)`` weights) the Q and K heads get
    the per-head RMS norm in the epilogue, and with ``rope`` (the model's
    ``(1, S, 1, 48, 2, 2)`` tensor, fp32 or bf16, whole sequence) also the
    split-half rotation of the chunk's rows."""
    lib = _native.load()
    rows, hidden = x_i8.shape
    n_out = w_i8.shape[0]
    if (x_i8.dtype != torch.int8 or w_i8.dtype != torch.int8 or not x_i8.is_contiguous() or not w_i8.is_contiguous()
            or w_i8.shape[1] != hidden):
        raise _native.NativeError("qkv_gemm_chunk: operands must be contiguous int8 with equal inner size")
    if (staging.dtype != torch.bfloat16 or staging.ndim != 3 or staging.shape[0] * HEAD_DIM != n_out
            or staging.shape[2] != HEAD_DIM or not staging.is_contiguous() or row_start + rows > staging.shape[1]):
        raise _native.NativeError("qkv_gemm_chunk: staging must be contiguous bf16 (n_out/128, S, 128) with room for the chunk")
    if x_scale.dtype != torch.float32 or w_scale.dtype != torch.float32 or x_scale.numel() < rows or w_scale.numel() != n_out:
        raise _native.NativeError("qkv_gemm_chunk: scales must be fp32 (rows,) and (n_out,)")
    base = ctypes.c_void_p(staging.data_ptr() + int(row_start) * HEAD_DIM * staging.element_size())
    if q_norm is None and k_norm is None and rope is None:
        check(
            lib.h3s_qkv_gemm_chunk(ptr(x_i8), ptr(x_scale), ptr(w_i8), ptr(w_scale), rows, hidden, n_out, base,
                                   staging.stride(0), ptr(status), stream_ptr(x_i8.device)),
            "h3s_qkv_gemm_chunk",
        )
        return
    if q_norm is None or k_norm is None:
        raise _native.NativeError("qkv_gemm_chunk: q_norm and k_norm go together (RoPE needs both)")
    if n_out % (3 * HEAD_DIM):
        raise _native.NativeError("qkv_gemm_chunk: n_out %d is not 3*heads*128" % n_out)
    for name, weight in (("q_norm", q_norm), ("k_norm", k_norm)):
        if weight.dtype != torch.float32 or tuple(weight.shape) != (HEAD_DIM,) or not weight.is_contiguous() \
                or weight.device != x_i8.device:
            raise _native.NativeError("qkv_gemm_chunk: %s must be a contiguous fp32 (128,) tensor on the GEMM's device" % name)
    rope_ptr, rope_code, strides = None, 0, None
    if rope is not None:
        sequence = staging.shape[1]
        if (rope.ndim != 6 or tuple(rope.shape[:3]) != (1, sequence, 1) or tuple(rope.shape[3:]) != (48, 2, 2)
                or rope.device != x_i8.device or rope.dtype not in (torch.float32, torch.bfloat16)):
            raise _native.NativeError("qkv_gemm_chunk: rope must be fp32/bf16 (1, %d, 1, 48, 2, 2) on the GEMM's device" % sequence)
        rope_ptr = ctypes.c_void_p(rope.data_ptr() + int(row_start) * rope.stride(1) * rope.element_size())
        rope_code = dtype_code(rope.dtype)
        strides = (ctypes.c_int64 * 4)(rope.stride(1), rope.stride(3), rope.stride(4), rope.stride(5))
    check(
        lib.h3s_qkv_gemm_chunk_norm_rope(
            ptr(x_i8), ptr(x_scale), ptr(w_i8), ptr(w_scale), rows, hidden, n_out // (3 * HEAD_DIM), base,
            staging.stride(0), ptr(q_norm), ptr(k_norm), float(epsilon), rope_ptr, rope_code, strides, ptr(status),
            stream_ptr(x_i8.device)),
        "h3s_qkv_gemm_chunk_norm_rope",
    )


def column_stats_scratch(heads, device):
    """Zeroed statistics scratch (K column sums in FP64, V column maxima) for
    ``qkv_gemm_chunk_carriers`` / ``column_stats_finalize``."""
    lib = _native.load()
    return torch.zeros(lib.h3s_column_stats_scratch_bytes(int(heads)), dtype=torch.uint8, device=device)


def column_stats_finalize(stats, heads, sequence, *, want_k_mean, dtype=torch.bfloat16, v_bound=FP8_V_BOUND):
    """``(k_mean | None, v_scale)`` from an accumulated statistics scratch."""
    lib = _native.load()
    k_mean = torch.empty((1, heads, HEAD_DIM), dtype=torch.float32, device=stats.device) if want_k_mean else None
    v_scale = torch.empty((1, heads, HEAD_DIM), dtype=torch.float32, device=stats.device)
    check(
        lib.h3s_column_stats_finalize(ptr(stats), dtype_code(dtype), int(heads), int(sequence), float(v_bound),
                                      ptr(k_mean), ptr(v_scale), stream_ptr(stats.device)),
        "h3s_column_stats_finalize",
    )
    return k_mean, v_scale


def qkv_gemm_chunk_carriers(x_i8, x_scale, w_i8, w_scale, *, heads, row_start, q_int8, q_scale, q_summary,
                            k_summary, v_stage, stats, k_int8=None, k_scale=None, k_stage=None, status=None,
                            q_norm=None, k_norm=None, epsilon=1e-6, rope=None):
    """INT8 GEMM of one chunk whose epilogue writes the carriers of rows
    ``[row_start, row_start + rows)``: INT8 Q blocks + scales + tile means, K
    either quantised the same way (``k_int8`` + ``k_scale``) or staged as bf16
    (``k_stage``) with its column sums accumulated in ``stats``, V staged as
    bf16 with its column maxima accumulated in ``stats``.  All output tensors
    cover the whole sequence."""
    lib = _native.load()
    rows, hidden = x_i8.shape
    sequence = q_int8.shape[2]
    n_out = 3 * heads * HEAD_DIM
    if (x_i8.dtype != torch.int8 or w_i8.dtype != torch.int8 or not x_i8.is_contiguous() or not w_i8.is_contiguous()
            or tuple(w_i8.shape) != (n_out, hidden)):
        raise _native.NativeError("qkv_gemm_chunk_carriers: operands must be contiguous int8, weight (3*heads*128, hidden)")
    if x_scale.dtype != torch.float32 or w_scale.dtype != torch.float32 or x_scale.numel() < rows or w_scale.numel() != n_out:
        raise _native.NativeError("qkv_gemm_chunk_carriers: scales must be fp32 (rows,) and (n_out,)")
    q_blocks, k_blocks = _ceil_div(sequence, Q_TILE), _ceil_div(sequence, KV_TILE)
    expect = [("q_int8", q_int8, (1, heads, sequence, HEAD_DIM), torch.int8),
              ("q_scale", q_scale, (1, heads, q_blocks), torch.float32),
              ("q_summary", q_summary, (1, heads, q_blocks, HEAD_DIM), None),
              ("k_summary", k_summary, (1, heads, k_blocks, HEAD_DIM), q_summary.dtype),
              ("v_stage", v_stage, (1, heads, sequence, HEAD_DIM), torch.bfloat16)]
    if k_stage is not None:
        expect.append(("k_stage", k_stage, (1, heads, sequence, HEAD_DIM), torch.bfloat16))
        if k_int8 is not None or k_scale is not None:
            raise _native.NativeError("qkv_gemm_chunk_carriers: K is either staged or quantised, not both")
    else:
        expect += [("k_int8", k_int8, (1, heads, sequence, HEAD_DIM), torch.int8),
                   ("k_scale", k_scale, (1, heads, k_blocks), torch.float32)]
    for name, t, shape, dt in expect:
        if t is None or tuple(t.shape) != shape or (dt is not None and t.dtype != dt) or not t.is_contiguous() \
                or t.device != x_i8.device:
            raise _native.NativeError("qkv_gemm_chunk_carriers: %s must be a contiguous %s tensor of shape %s on the GEMM's device"
                                      % (name, dt, shape))
    carriers = _native.QKVCarriers(
        q8=q_int8.data_ptr(), q_scale=q_scale.data_ptr(), q_summary=q_summary.data_ptr(),
        k8=None if k_int8 is None else k_int8.data_ptr(), k_scale=None if k_scale is None else k_scale.data_ptr(),
        k_summary=k_summary.data_ptr(), k_stage=None if k_stage is None else k_stage.data_ptr(),
        v_stage=v_stage.data_ptr(), stats=stats.data_ptr(), summary_dtype=dtype_code(q_summary.dtype),
        sequence_total=int(sequence), row_start=int(row_start),
    )
    if (q_norm is None) != (k_norm is None):
        raise _native.NativeError("qkv_gemm_chunk_carriers: q_norm and k_norm go together")
    if rope is not None and q_norm is None:
        raise _native.NativeError("qkv_gemm_chunk_carriers: the rotation needs the norm weights")
    rope_ptr, rope_code, strides = None, 0, None
    if rope is not None:
        if (rope.ndim != 6 or tuple(rope.shape[:3]) != (1, sequence, 1) or tuple(rope.shape[3:]) != (48, 2, 2)
                or rope.device != x_i8.device or rope.dtype not in (torch.float32, torch.bfloat16)):
            raise _native.NativeError("qkv_gemm_chunk_carriers: rope must be fp32/bf16 (1, %d, 1, 48, 2, 2) on the GEMM's device" % sequence)
        rope_ptr = ctypes.c_void_p(rope.data_ptr() + int(row_start) * rope.stride(1) * rope.element_size())
        rope_code = dtype_code(rope.dtype)
        strides = (ctypes.c_int64 * 4)(rope.stride(1), rope.stride(3), rope.stride(4), rope.stride(5))
    check(
        lib.h3s_qkv_gemm_chunk_carriers(
            ptr(x_i8), ptr(x_scale), ptr(w_i8), ptr(w_scale), rows, hidden, int(heads), ctypes.byref(carriers),
            ptr(q_norm), ptr(k_norm), float(epsilon), rope_ptr, rope_code, strides, ptr(status),
            stream_ptr(x_i8.device)),
        "h3s_qkv_gemm_chunk_carriers",
    )


GEMM_KINDS = {torch.int8: 0, torch.bfloat16: 1, torch.float16: 2, torch.float8_e4m3fn: 3}
ACT_NONE, ACT_GELU_TANH = 0, 1


def dense_gemm(a, b, *, row_scale=None, col_scale=None, bias=None, activation="none", out=None, status=None):
    """``out = bf16(act((a @ b.T) * row_scale[:, None] * col_scale[None, :] + bias))`` on the
    tensor cores.  ``a`` (rows, K) and ``b`` (n_out, K) share one element type
    (int8, bf16, fp16 or float8_e4m3fn) and have contiguous rows; ``b`` is a
    Linear weight as stored.  ``activation``: ``"none"`` or ``"gelu_tanh"``."""
    lib = _native.load()
    if a.ndim != 2 or b.ndim != 2 or a.shape[1] != b.shape[1] or a.dtype != b.dtype or a.dtype not in GEMM_KINDS:
        raise _native.NativeError("dense_gemm: a (rows, K) and b (n_out, K) must share K and an int8/bf16/fp16/e4m3 type")
    if not (a.is_cuda and b.is_cuda) or a.stride(1) != 1 or b.stride(1) != 1:
        raise _native.NativeError("dense_gemm: operands must be CUDA tensors with contiguous rows")
    rows, k = a.shape
    n_out = b.shape[0]
    if out is None:
        out = torch.empty((rows, n_out), dtype=torch.bfloat16, device=a.device)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (rows, n_out) or out.stride(1) != 1:
        raise _native.NativeError("dense_gemm: out must be bf16 (rows, n_out) with contiguous rows")
    for name, t, n in (("row_scale", row_scale, rows), ("col_scale", col_scale, n_out), ("bias", bias, n_out)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous() or t.device != a.device):
            raise _native.NativeError("dense_gemm: %s must be a contiguous fp32 tensor of %d elements on the operands' device" % (name, n))
    act = {"none": ACT_NONE, "gelu_tanh": ACT_GELU_TANH}.get(activation)
    if act is None:
        raise _native.NativeError("dense_gemm: activation must be 'none' or 'gelu_tanh'")
    size = a.element_size()
    check(
        lib.h3s_dense_gemm(ptr(a), a.stride(0) * size, ptr(b), b.stride(0) * size, GEMM_KINDS[a.dtype], rows, n_out,
                           k * size, ptr(row_scale), ptr(col_scale), ptr(bias), act, ptr(out), out.stride(0),
                           ptr(status), stream_ptr(a.device)),
        "h3s_dense_gemm",
    )
    return out


def quant_rows_fp8(x, out=None, row_scale=None):
    """Per-row FP8-E4M3 of a bf16 matrix: ``(codes e4m3 (rows, C), scale fp32 (rows,))``."""
    lib = _native.load()
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_cuda or x.stride(1) != 1:
        raise _native.NativeError("quant_rows_fp8: x must be a rank-2 CUDA bf16 tensor with contiguous rows")
    rows, channels = x.shape
    if out is None:
        out = torch.empty((rows, channels), dtype=torch.float8_e4m3fn, device=x.device)
    if row_scale is None:
        row_scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
    if out.shape[0] < rows or out.shape[1] != channels or not out.is_contiguous() or row_scale.numel() < rows:
        raise _native.NativeError("quant_rows_fp8: output buffers are too small")
    check(lib.h3s_quant_rows_fp8(ptr(x), x.stride(0), rows, channels, ptr(out), ptr(row_scale), stream_ptr(x.device)),
          "h3s_quant_rows_fp8")
    return out[:rows], row_scale[:rows]


def route_topk(q_summary, k_summary, *, q_start, q_stop, kv_start, kv_stop, retained):
    """Compact route ``int32 (1,H,q_stop-q_start,route_len)``."""
    lib = _native.load()
    if q_summary.ndim != 4 or k_summary.ndim != 4 or q_summary.shape[0] != 1:
        raise _native.NativeError("route_topk: summaries must be rank-4 (1,H,tiles,128)")
    if q_summary.dtype != k_summary.dtype:
        raise _native.NativeError("route_topk: summary dtypes differ")
    q_summary = q_summary.contiguous()
    k_summary = k_summary.contiguous()
    heads, q_tiles = q_summary.shape[1], q_summary.shape[2]
    kv_tiles = k_summary.shape[2]
    route_len = kv_tiles - (kv_stop - kv_start) + retained
    route = torch.empty((1, heads, q_stop - q_start, route_len), dtype=torch.int32, device=q_summary.device)
    check(
        lib.h3s_route_topk(
            ptr(q_summary), ptr(k_summary), dtype_code(q_summary.dtype), heads, q_tiles, kv_tiles,
            int(q_start), int(q_stop), int(kv_start), int(kv_stop), int(retained), ptr(route),
            stream_ptr(q_summary.device),
        ),
        "h3s_route_topk",
    )
    return route


def route_to_delta_lut(route, *, heads, q_tiles, kv_tiles, q_start, q_stop, device):
    lib = _native.load()
    lut = torch.empty((1, heads, q_tiles, kv_tiles), dtype=torch.int32, device=device)
    valid = torch.empty((1, heads, q_tiles), dtype=torch.int32, device=device)
    route_len = 0 if route is None else route.shape[-1]
    check(
        lib.h3s_route_to_delta_lut(
            ptr(route), heads, q_tiles, kv_tiles, int(q_start), int(q_stop), int(route_len), ptr(lut),
            ptr(valid), stream_ptr(device),
        ),
        "h3s_route_to_delta_lut",
    )
    return lut, valid


def _attn_args(q8, k8, v_carrier, q_scale, k_scale, v_scale, route, q_start, q_stop, out):
    heads, sequence = q8.shape[1], q8.shape[2]
    for name, t, dt in (("q8", q8, torch.int8), ("k8", k8, torch.int8), ("v_carrier", v_carrier, torch.float8_e4m3fn),
                        ("q_scale", q_scale, torch.float32), ("k_scale", k_scale, torch.float32),
                        ("v_scale", v_scale, torch.float32)):
        if t.dtype != dt or not t.is_contiguous() or not t.is_cuda:
            raise _native.NativeError("sparse_attention: %s must be a contiguous CUDA %s tensor" % (name, dt))
    padded = _ceil_div(sequence, 128) * 128
    if tuple(k8.shape) != tuple(q8.shape) or tuple(v_carrier.shape) != (1, heads, HEAD_DIM, padded):
        raise _native.NativeError("sparse_attention: carrier shapes do not agree")
    if (tuple(q_scale.shape) != (1, heads, _ceil_div(sequence, Q_TILE))
            or tuple(k_scale.shape) != (1, heads, _ceil_div(sequence, KV_TILE))
            or tuple(v_scale.shape) != (1, heads, HEAD_DIM)):
        raise _native.NativeError("sparse_attention: scale shapes do not agree")
    route_len = 0
    if route is not None:
        if route.dtype != torch.int32 or not route.is_contiguous() or tuple(route.shape[:3]) != (1, heads, q_stop - q_start):
            raise _native.NativeError("sparse_attention: route must be contiguous int32 (1,H,%d,len)" % (q_stop - q_start))
        route_len = route.shape[-1]
    if out.shape != q8.shape or out.stride(-1) != 1:
        raise _native.NativeError("sparse_attention: output must be (1,H,S,128) with a contiguous last dimension")
    return heads, sequence, route_len


def new_attention_output(heads, sequence, dtype, device):
    """HND view of a token-major ``(S, H*128)`` buffer, so the caller's
    transpose+reshape before ``out_proj`` (attention_forward.py:123-128) is free."""
    base = torch.empty((1, sequence, heads, HEAD_DIM), dtype=dtype, device=device)
    return base.permute(0, 2, 1, 3)


def sparse_attention(q8, k8, v_carrier, q_scale, k_scale, v_scale, route=None, *, q_start=0, q_stop=0,
                     out=None, out_dtype=torch.bfloat16, status=None, legacy_mma=False, single_term_p=False,
                     peer_out_ptrs=None, extra_flags=0):
    """Launch the attention kernel.  Returns ``out`` (HND).  ``single_term_p``
    carries the probabilities as one E4M3 term instead of hi + lo.
    ``peer_out_ptrs``: device addresses (ints) of up to 7 further buffers,
    addressed like ``out``, that receive every output tile as well (the slices
    of the peer GPUs' full outputs in a head-sharded run)."""
    lib = _native.load()
    if out is None:
        out = new_attention_output(q8.shape[1], q8.shape[2], out_dtype, q8.device)
    heads, sequence, route_len = _attn_args(q8, k8, v_carrier, q_scale, k_scale, v_scale, route, q_start, q_stop, out)
    common = (
        ptr(q8), ptr(k8), ptr(v_carrier), ptr(q_scale), ptr(k_scale), ptr(v_scale), ptr(route), route_len,
        int(q_start), int(q_stop), ptr(out), dtype_code(out.dtype), out.stride(1), out.stride(2), heads, sequence,
    )
    flags = (ATTN_P_SINGLE if single_term_p else 0) | int(extra_flags)
    if peer_out_ptrs:
        if legacy_mma:
            raise _native.NativeError("sparse_attention: the cross-check kernel does not scatter to peers")
        table = (ctypes.c_void_p * len(peer_out_ptrs))(*[ctypes.c_void_p(int(p)) for p in peer_out_ptrs])
        check(
            lib.h3s_sparse_attn_fwd_scatter(*common[:11], table, len(peer_out_ptrs), *common[11:], flags,
                                            ptr(status), stream_ptr(q8.device)),
            "h3s_sparse_attn_fwd_scatter",
        )
        return out
    if legacy_mma:
        check(lib.h3s_sparse_attn_fwd_mma(*common, flags, stream_ptr(q8.device)), "h3s_sparse_attn_fwd_mma")
    else:
        check(lib.h3s_sparse_attn_fwd(*common, flags, ptr(status), stream_ptr(q8.device)), "h3s_sparse_attn_fwd")
    return out
