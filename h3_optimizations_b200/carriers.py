"""Carrier data contracts (reference: attention/sparse/fused_qkv.py:30-154,
attention/sparse/sparse_sage.py:401-417)."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .errors import FusedQKVError
from .router import KV_TILE, Q_TILE

HEAD_DIM = 128


@dataclass
class PreparedFusedQKV:
    """Output of a QKV projector: INT8 Q/K carriers with per-block scales and
    tile means, plus V either floating HND (``v``) or already packed
    (``v_carrier`` e4m3 ``(1,H,128,pad128(S))`` + ``v_scale`` ``(1,H,128)``)."""

    q_int8: torch.Tensor
    q_scale: torch.Tensor
    k_int8: torch.Tensor
    k_scale: torch.Tensor
    v: torch.Tensor | None
    q_summary: torch.Tensor
    k_summary: torch.Tensor
    output_dtype: torch.dtype
    sequence: int
    heads: int
    head_dim: int
    layer_index: int
    smooth_k: bool = False
    v_carrier: torch.Tensor | None = None
    v_scale: torch.Tensor | None = None


def validate_prepared_fused_qkv(prepared):
    sequence = int(prepared.sequence)
    heads = int(prepared.heads)
    head_dim = int(prepared.head_dim)
    shape = (1, heads, sequence, head_dim)
    q_blocks = (sequence + Q_TILE - 1) // Q_TILE
    k_blocks = (sequence + KV_TILE - 1) // KV_TILE
    if head_dim != HEAD_DIM:
        raise FusedQKVError("fused H3 QKV requires head_dim 128")
    if tuple(prepared.q_int8.shape) != shape or tuple(prepared.k_int8.shape) != shape:
        raise FusedQKVError("fused H3 Q/K carrier shape is invalid")
    if prepared.q_int8.dtype != torch.int8 or prepared.k_int8.dtype != torch.int8:
        raise FusedQKVError("fused H3 Q/K carriers must be INT8")
    if prepared.v_carrier is None:
        if prepared.v is None:
            raise FusedQKVError("fused H3 V is missing")
        if tuple(prepared.v.shape) != shape or prepared.v.dtype != prepared.output_dtype:
            raise FusedQKVError("fused H3 V carrier is invalid")
    else:
        padded = (sequence + 127) // 128 * 128
        if tuple(prepared.v_carrier.shape) != (1, heads, head_dim, padded):
            raise FusedQKVError("prepacked H3 FP8 V carrier shape is invalid")
        if prepared.v_carrier.dtype != torch.float8_e4m3fn:
            raise FusedQKVError("prepacked H3 V carrier must be E4M3 FP8")
        if prepared.v_scale is None:
            raise FusedQKVError("prepacked H3 FP8 V requires V scale")
        if tuple(prepared.v_scale.shape) != (1, heads, head_dim):
            raise FusedQKVError("prepacked H3 V scale shape is invalid")
        if prepared.v_scale.dtype != torch.float32:
            raise FusedQKVError("prepacked H3 V scale must be FP32")
    if tuple(prepared.q_scale.shape) != (1, heads, q_blocks):
        raise FusedQKVError("fused H3 Q scale shape is invalid")
    if tuple(prepared.k_scale.shape) != (1, heads, k_blocks):
        raise FusedQKVError("fused H3 K scale shape is invalid")
    if prepared.q_scale.dtype != torch.float32 or prepared.k_scale.dtype != torch.float32:
        raise FusedQKVError("fused H3 Q/K scales must be float32")
    if tuple(prepared.q_summary.shape) != (1, heads, q_blocks, head_dim):
        raise FusedQKVError("fused H3 Q router summary shape is invalid")
    if tuple(prepared.k_summary.shape) != (1, heads, k_blocks, head_dim):
        raise FusedQKVError("fused H3 K router summary shape is invalid")
    tensors = [prepared.q_int8, prepared.q_scale, prepared.k_int8, prepared.k_scale,
               prepared.q_summary, prepared.k_summary]
    for extra in (prepared.v, prepared.v_carrier, prepared.v_scale):
        if extra is not None:
            tensors.append(extra)
    if any(t.device != prepared.q_int8.device for t in tensors):
        raise FusedQKVError("fused H3 QKV carrier devices differ")
    contiguous = [t for t in tensors if t is not prepared.v]
    if any(not t.is_contiguous() for t in contiguous):
        raise FusedQKVError("fused H3 QKV carriers must be contiguous")
    return prepared


@dataclass
class PreparedSparse:
    """Everything one attention launch needs (the counterpart of
    ``PreparedSparseSage``): carriers, scales, the packed route and metadata.
    ``lut`` / ``valid_block_num`` in the reference's delta encoding are
    produced on demand by ``B200SparseBackend.reference_lut``."""

    q_int8: torch.Tensor
    k_int8: torch.Tensor
    v_carrier: torch.Tensor
    q_scale: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor
    route: object  # router.SparseRoute
    output_dtype: torch.dtype
    output_shape: tuple
    layer_index: int
    sequence: int
    heads: int
    metadata: dict = field(default_factory=dict)


@dataclass
class PreparedHybrid:
    sparse: PreparedSparse
