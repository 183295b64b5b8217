"""``torch.library`` custom operators over the C ABI, with fake (meta)
implementations, so that a graph tracer (``torch.compile``, fake-tensor
propagation) sees the hot path as opaque operators with known output shapes
instead of ctypes calls.

The reference registers its operators the same way and under the pack's
``h3_optimizations::`` namespace (attention/sparse/router.py:18-29,
sparse_sage.py:354-398, fused_qkv.py:615-690; tests/test_source_isolation.py:
31-40 insists on the namespace).  The operators here carry a ``b200_`` prefix
so that both sets can be loaded into one process:

* ``h3_optimizations::b200_quantize_qk_blocks(x, block, mean?) -> (codes, scale, summary)``
* ``h3_optimizations::b200_prepare_v(v) -> (carrier, scale)``
  (shapes as ``prepare_sparse_sage_v``, sparse_sage.py:354-367)
* ``h3_optimizations::b200_route(q_summary, k_summary, q_start, q_stop, kv_start, kv_stop, retained) -> route``
* ``h3_optimizations::b200_sparse_attention(q_int8, k_int8, v_carrier, route, q_scale, k_scale, v_scale,
  q_start, q_stop, output_dtype) -> out``  (counterpart of ``sparse_sage_attention``, sparse_sage.py:372-398)

Importing this module registers the operators; the real implementations are
CUDA-only and raise like the plain wrappers in ``ops`` when the native library
or a B200 is missing.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops

NAMESPACE = "h3_optimizations"
HEAD_DIM = 128


@torch.library.custom_op(NAMESPACE + "::b200_quantize_qk_blocks", mutates_args=(), device_types="cuda")
def quantize_qk_blocks_op(x: torch.Tensor, block: int, mean: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    codes, scale, summary = ops.quant_qk_blocks(x, block, mean=mean, summary_dtype=torch.float64)
    return codes, scale, summary


@quantize_qk_blocks_op.register_fake
def _quantize_qk_blocks_fake(x, block, mean):
    blocks = (x.shape[-2] + block - 1) // block
    return (x.new_empty(x.shape, dtype=torch.int8),
            x.new_empty((*x.shape[:-2], blocks), dtype=torch.float32),
            x.new_empty((*x.shape[:-2], blocks, x.shape[-1]), dtype=torch.float64))


@torch.library.custom_op(NAMESPACE + "::b200_prepare_v", mutates_args=(), device_types="cuda")
def prepare_v_op(v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    carrier, scale = ops.quant_v_fp8(v)
    return carrier, scale


@prepare_v_op.register_fake
def _prepare_v_fake(v):
    padded = (v.shape[-2] + 127) // 128 * 128
    return (v.new_empty((*v.shape[:-2], v.shape[-1], padded), dtype=torch.float8_e4m3fn),
            v.new_empty((*v.shape[:-2], v.shape[-1]), dtype=torch.float32))


@torch.library.custom_op(NAMESPACE + "::b200_route", mutates_args=(), device_types="cuda")
def route_op(q_summary: torch.Tensor, k_summary: torch.Tensor, q_start: int, q_stop: int, kv_start: int,
             kv_stop: int, retained: int) -> torch.Tensor:
    return ops.route_topk(q_summary, k_summary, q_start=q_start, q_stop=q_stop, kv_start=kv_start,
                          kv_stop=kv_stop, retained=retained)


@route_op.register_fake
def _route_fake(q_summary, k_summary, q_start, q_stop, kv_start, kv_stop, retained):
    route_len = k_summary.shape[-2] - (kv_stop - kv_start) + retained
    return q_summary.new_empty((*q_summary.shape[:-2], q_stop - q_start, route_len), dtype=torch.int32)


@torch.library.custom_op(NAMESPACE + "::b200_sparse_attention", mutates_args=(), device_types="cuda")
def sparse_attention_op(q_int8: torch.Tensor, k_int8: torch.Tensor, v_carrier: torch.Tensor,
                        route: Optional[torch.Tensor], q_scale: torch.Tensor, k_scale: torch.Tensor,
                        v_scale: torch.Tensor, q_start: int, q_stop: int,
                        output_dtype: torch.dtype) -> torch.Tensor:
    out = torch.empty(q_int8.shape, dtype=output_dtype, device=q_int8.device)
    ops.sparse_attention(q_int8, k_int8, v_carrier, q_scale, k_scale, v_scale, route, q_start=q_start,
                         q_stop=q_stop, out=out)
    return out


@sparse_attention_op.register_fake
def _sparse_attention_fake(q_int8, k_int8, v_carrier, route, q_scale, k_scale, v_scale, q_start, q_stop,
                           output_dtype):
    return q_int8.new_empty(q_int8.shape, dtype=output_dtype)


def quantize_qk_blocks(x, block, mean=None):
    return quantize_qk_blocks_op(x, int(block), mean)


def prepare_v(v):
    return prepare_v_op(v)


def route(q_summary, k_summary, *, q_start, q_stop, kv_start, kv_stop, retained):
    return route_op(q_summary, k_summary, int(q_start), int(q_stop), int(kv_start), int(kv_stop), int(retained))


def sparse_attention(q_int8, k_int8, v_carrier, route, q_scale, k_scale, v_scale, *, q_start=0, q_stop=0,
                     output_dtype=torch.bfloat16):
    return sparse_attention_op(q_int8, k_int8, v_carrier, route, q_scale, k_scale, v_scale, int(q_start),
                               int(q_stop), output_dtype)
