"""Chunked native-carrier QKV provider for the B200 backend.

Counterpart of the reference's ``ChunkedSparseQKVProjector``
(attention/sparse/chunked_qkv.py:205-366): the packed ``x (S, hidden)`` is
projected in 4096-row chunks straight into full-length quantised carriers, so
no full-precision Q/K/V of the whole sequence is handed to the backend.

Per chunk:  ConvRot (Hadamard-256) + per-row INT8 of the activations
            -> tcgen05 INT8 GEMM against the INT8 QKV weight whose epilogue
               writes the carriers: INT8 Q blocks, scales and tile means
               straight from the accumulators (Q is never stored in a wider
               format), K tile means, bf16 staging of K and V with their
               column sums / maxima accumulated on the way.
After the last chunk (K smoothing and the V scale need whole-sequence
statistics): the statistics are finalised, the staged K is quantised with the
mean removed and the staged V becomes the FP8-E4M3 carrier.  With
``smooth_k=False`` (what every chunked producer of the reference does,
chunked_qkv.py:289) K leaves the epilogue as INT8 blocks like Q and only V is
staged.  The default keeps the smoothing on, which is what the attention
kernel's accuracy figures are stated for.

The module handed to ``project`` must expose ``heads``, ``head_dim`` and the
INT8 weight in the rotated domain: ``qkv_weight_int8`` (3*H*128, hidden) with
rows ordered ``[Q heads | K heads | V heads]`` (fused_qkv.py:195,394) and
``qkv_weight_scale`` (3*H*128,) fp32.  When the module carries ``q_norm`` and
``k_norm`` (objects with ``weight`` (128,) and ``eps``) the per-head RMS norm of
Q and K runs in the GEMM epilogue, and with ``rope_freqs`` (1,S,1,48,2,2) the
split-half rotation as well (fused_qkv.py:225-289); a module without norms
(the benchmark configuration) is projected without either, and asking for the
rotation without norms is an error.
"""

from __future__ import annotations

import math

import torch

from . import _native, ops
from .carriers import PreparedFusedQKV, validate_prepared_fused_qkv
from .errors import FusedQKVError
from .router import KV_TILE, Q_TILE

CHUNK_ROWS = 4096
HEAD_DIM = 128
V_QUANT_BOUND = 448.0


_SIDE_STREAMS = {}


def _side_stream(device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device)
    return _SIDE_STREAMS[key]


def _validate_chunk_rows(chunk_rows, q_tile=Q_TILE, kv_tile=KV_TILE):
    chunk_rows = int(chunk_rows)
    alignment = math.lcm(int(q_tile), int(kv_tile))
    if chunk_rows <= 0 or chunk_rows % alignment:
        raise FusedQKVError(
            "chunked Sparse Sage QKV rows must be a positive multiple of %d" % alignment
        )
    return chunk_rows


def chunk_ranges(sequence, chunk_rows):
    return [(start, min(start + chunk_rows, sequence)) for start in range(0, sequence, chunk_rows)]


class ChunkedSparseQKVProjector:
    name = "chunked_b200_sparse_qkv"
    qk_format = "sparge_block_int8"

    def __init__(self, chunk_rows=CHUNK_ROWS, *, smooth_k=True, summary_dtype=torch.float32):
        self.chunk_rows = _validate_chunk_rows(chunk_rows)
        self.smooth_k = bool(smooth_k)
        self.summary_dtype = summary_dtype

    @property
    def installation_signature(self):
        return (self.name, self.qk_format, self.chunk_rows, ("sm_100a", _native.ABI_VERSION, self.smooth_k))

    # -- protocol ---------------------------------------------------------

    def try_project(self, module, x, rope_freqs, *, layer_index, transformer_options):
        if rope_freqs is not None and (getattr(module, "q_norm", None) is None or getattr(module, "k_norm", None) is None):
            return None
        if getattr(module, "qkv_weight_int8", None) is None or getattr(module, "qkv_weight_scale", None) is None:
            return None
        return self.project(module, x, rope_freqs, layer_index=layer_index, transformer_options=transformer_options)

    def project(self, module, x, rope_freqs, *, layer_index, transformer_options):
        del transformer_options
        weight = getattr(module, "qkv_weight_int8", None)
        scale = getattr(module, "qkv_weight_scale", None)
        if weight is None or scale is None:
            raise FusedQKVError("module does not expose qkv_weight_int8 / qkv_weight_scale")
        q_norm, k_norm = getattr(module, "q_norm", None), getattr(module, "k_norm", None)
        if (q_norm is None) != (k_norm is None):
            raise FusedQKVError("module must carry both q_norm and k_norm or neither")
        if rope_freqs is not None and q_norm is None:
            raise FusedQKVError("RoPE in the QKV epilogue needs the module's q_norm / k_norm")
        norm = None
        if q_norm is not None:
            if float(q_norm.eps) != float(k_norm.eps):
                raise FusedQKVError("q_norm and k_norm use different epsilons")
            norm = (q_norm.weight, k_norm.weight, float(q_norm.eps))
        return run_chunked_sparse_qkv(
            x, weight, scale, heads=int(module.heads), head_dim=int(module.head_dim),
            layer_index=layer_index, chunk_rows=self.chunk_rows, smooth_k=self.smooth_k,
            summary_dtype=self.summary_dtype, norm=norm, rope_freqs=rope_freqs,
        )


def run_chunked_sparse_qkv(x, w_i8, w_scale, *, heads, head_dim=HEAD_DIM, layer_index=0,
                           chunk_rows=CHUNK_ROWS, smooth_k=True, summary_dtype=torch.float32,
                           status=None, norm=None, rope_freqs=None):
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.ndim != 2:
        raise FusedQKVError("chunked Sparse Sage QKV requires a rank-2 CUDA BF16 input")
    if torch.is_grad_enabled() and x.requires_grad:
        raise FusedQKVError("chunked Sparse Sage QKV is inference-only")
    if head_dim != HEAD_DIM:
        raise FusedQKVError("chunked Sparse Sage QKV requires H3 head_dim 128")
    chunk_rows = _validate_chunk_rows(chunk_rows)
    sequence, hidden = int(x.shape[0]), int(x.shape[1])
    n_out = 3 * heads * HEAD_DIM
    if sequence <= 0 or tuple(w_i8.shape) != (n_out, hidden) or w_i8.dtype != torch.int8:
        raise FusedQKVError("QKV weight must be int8 (3*heads*128, hidden) = (%d, %d)" % (n_out, hidden))
    if tuple(w_scale.shape) != (n_out,) or w_scale.dtype != torch.float32:
        raise FusedQKVError("QKV weight scale must be fp32 (%d,)" % n_out)
    device = x.device
    q_norm = k_norm = None
    epsilon = 0.0
    if norm is not None:
        q_norm, k_norm, epsilon = norm
        q_norm = q_norm.detach().to(device=device, dtype=torch.float32).contiguous()
        k_norm = k_norm.detach().to(device=device, dtype=torch.float32).contiguous()
        if tuple(q_norm.shape) != (HEAD_DIM,) or tuple(k_norm.shape) != (HEAD_DIM,):
            raise FusedQKVError("q_norm / k_norm weights must have 128 elements")
    if rope_freqs is not None:
        if norm is None:
            raise FusedQKVError("RoPE in the QKV epilogue needs the q_norm / k_norm weights")
        if (rope_freqs.ndim != 6 or tuple(rope_freqs.shape[:3]) != (1, sequence, 1)
                or tuple(rope_freqs.shape[3:]) != (48, 2, 2) or rope_freqs.device != device):
            raise FusedQKVError("rope_freqs must be (1, %d, 1, 48, 2, 2) on the projection's device" % sequence)
        if rope_freqs.dtype not in (torch.float32, torch.bfloat16):
            rope_freqs = rope_freqs.float()
    try:
        q_blocks = (sequence + Q_TILE - 1) // Q_TILE
        k_blocks = (sequence + KV_TILE - 1) // KV_TILE
        shape = (1, heads, sequence, HEAD_DIM)
        q_int8 = torch.empty(shape, dtype=torch.int8, device=device)
        k_int8 = torch.empty(shape, dtype=torch.int8, device=device)
        q_scale = torch.empty((1, heads, q_blocks), dtype=torch.float32, device=device)
        k_scale = torch.empty((1, heads, k_blocks), dtype=torch.float32, device=device)
        q_summary = torch.empty((1, heads, q_blocks, HEAD_DIM), dtype=summary_dtype, device=device)
        k_summary = torch.empty((1, heads, k_blocks, HEAD_DIM), dtype=summary_dtype, device=device)
        # bf16 staging of what needs whole-sequence statistics before it can be quantised
        v_stage = torch.empty(shape, dtype=torch.bfloat16, device=device)
        k_stage = torch.empty(shape, dtype=torch.bfloat16, device=device) if smooth_k else None
        stats = ops.column_stats_scratch(heads, device)
        x_i8 = torch.empty((min(chunk_rows, sequence), hidden), dtype=torch.int8, device=device)
        x_scale = torch.empty((min(chunk_rows, sequence),), dtype=torch.float32, device=device)
        w_i8 = w_i8.contiguous()
        for start, end in chunk_ranges(sequence, chunk_rows):
            rows = end - start
            ops.convrot_quant_rows(x[start:end], x_i8, x_scale)
            ops.qkv_gemm_chunk_carriers(
                x_i8[:rows], x_scale[:rows], w_i8, w_scale, heads=heads, row_start=start,
                q_int8=q_int8, q_scale=q_scale, q_summary=q_summary, k_summary=k_summary, v_stage=v_stage,
                stats=stats, k_int8=None if smooth_k else k_int8, k_scale=None if smooth_k else k_scale,
                k_stage=k_stage, status=status, q_norm=q_norm, k_norm=k_norm, epsilon=epsilon, rope=rope_freqs)
        k_mean, v_scale = ops.column_stats_finalize(stats, heads, sequence, want_k_mean=smooth_k,
                                                    dtype=torch.bfloat16, v_bound=V_QUANT_BOUND)
        v_carrier = ops.allocate_v_carrier(sequence, heads, device)
        if smooth_k:
            # the two second-phase quantisers are independent and each leaves part of the
            # memory system idle: V runs on a second stream underneath K
            main, side = torch.cuda.current_stream(device), _side_stream(device)
            side.wait_stream(main)
            try:
                with torch.cuda.stream(side):
                    ops.quant_v_fp8_into(v_stage, v_scale, v_carrier, v_bound=V_QUANT_BOUND)
                ops.quant_qk_blocks_into(k_stage, k_int8, k_scale, None, block=KV_TILE, mean=k_mean)
            finally:
                main.wait_stream(side)  # on every exit path, before the staging can be freed
        else:
            ops.quant_v_fp8_into(v_stage, v_scale, v_carrier, v_bound=V_QUANT_BOUND)
    except _native.NativeError as exc:
        raise FusedQKVError("chunked QKV projection failed: layer=%d: %s" % (layer_index, exc)) from exc
    return validate_prepared_fused_qkv(
        PreparedFusedQKV(
            q_int8=q_int8, q_scale=q_scale, k_int8=k_int8, k_scale=k_scale, v=None,
            q_summary=q_summary, k_summary=k_summary, output_dtype=x.dtype, sequence=sequence,
            heads=heads, head_dim=HEAD_DIM, layer_index=int(layer_index), smooth_k=bool(smooth_k),
            v_carrier=v_carrier, v_scale=v_scale,
        )
    )
