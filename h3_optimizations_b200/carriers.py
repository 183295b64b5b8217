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


def _carrier_spec(prepared):
    """What each tensor of a ``PreparedFusedQKV`` must look like, as rows of
    ``(field, tensor, shape, dtype | None, message)``, in the order they are checked."""
    sequence, heads, head_dim = int(prepared.sequence), int(prepared.heads), int(prepared.head_dim)
    q_blocks, k_blocks = -(-sequence // Q_TILE), -(-sequence // KV_TILE)
    full = (1, heads, sequence, head_dim)
    rows = [
        ("q_int8", prepared.q_int8, full, None, "fused H3 Q/K carrier shape is invalid"),
        ("k_int8", prepared.k_int8, full, None, "fused H3 Q/K carrier shape is invalid"),
        ("q_int8", prepared.q_int8, None, torch.int8, "fused H3 Q/K carriers must be INT8"),
        ("k_int8", prepared.k_int8, None, torch.int8, "fused H3 Q/K carriers must be INT8"),
    ]
    if prepared.v_carrier is None:
        if prepared.v is None:
            raise FusedQKVError("fused H3 V is missing")
        rows.append(("v", prepared.v, full, prepared.output_dtype, "fused H3 V carrier is invalid"))
    else:
        padded = -(-sequence // 128) * 128
        rows.append(("v_carrier", prepared.v_carrier, (1, heads, head_dim, padded), None,
                     "prepacked H3 FP8 V carrier shape is invalid"))
        rows.append(("v_carrier", prepared.v_carrier, None, torch.float8_e4m3fn, "prepacked H3 V carrier must be E4M3 FP8"))
        if prepared.v_scale is None:
            raise FusedQKVError("prepacked H3 FP8 V requires V scale")
        rows.append(("v_scale", prepared.v_scale, (1, heads, head_dim), None, "prepacked H3 V scale shape is invalid"))
        rows.append(("v_scale", prepared.v_scale, None, torch.float32, "prepacked H3 V scale must be FP32"))
    rows += [
        ("q_scale", prepared.q_scale, (1, heads, q_blocks), None, "fused H3 Q scale shape is invalid"),
        ("k_scale", prepared.k_scale, (1, heads, k_blocks), None, "fused H3 K scale shape is invalid"),
        ("q_scale", prepared.q_scale, None, torch.float32, "fused H3 Q/K scales must be float32"),
        ("k_scale", prepared.k_scale, None, torch.float32, "fused H3 Q/K scales must be float32"),
        ("q_summary", prepared.q_summary, (1, heads, q_blocks, head_dim), None, "fused H3 Q router summary shape is invalid"),
        ("k_summary", prepared.k_summary, (1, heads, k_blocks, head_dim), None, "fused H3 K router summary shape is invalid"),
    ]
    return rows


def validate_prepared_fused_qkv(prepared):
    """Check a projector's output against the carrier contract
    (attention/sparse/fused_qkv.py:95-154: same conditions, same
    ``FusedQKVError`` texts) and hand it back.  The conditions are a table
    (``_carrier_spec``) walked once; device and contiguity are checked over
    every tensor the table names."""
    if int(prepared.head_dim) != HEAD_DIM:
        raise FusedQKVError("fused H3 QKV requires head_dim 128")
    seen = {}
    for name, tensor, shape, dtype, message in _carrier_spec(prepared):
        if shape is not None and tuple(tensor.shape) != shape:
            raise FusedQKVError(message)
        if dtype is not None and tensor.dtype != dtype:
            raise FusedQKVError(message)
        seen[name] = tensor
    home = prepared.q_int8.device
    if any(tensor.device != home for tensor in seen.values()):
        raise FusedQKVError("fused H3 QKV carrier devices differ")
    # V in floating point may be a strided view of the projection; everything else is dense
    if any(not tensor.is_contiguous() for name, tensor in seen.items() if name != "v"):
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
