"""torch.library operators on the device: same results as the plain wrappers."""

import pytest
import torch

from h3_optimizations_b200 import workloads

pytestmark = pytest.mark.gpu


def test_registered_ops_match_the_plain_wrappers(native_lib):
    from h3_optimizations_b200 import ops, torch_ops

    spec = workloads.small_spec("ops", 2, 256, 1024)
    q, k, v = (t.cuda() for t in workloads.gaussian_qkv(spec, seed=2))
    k_mean, _ = ops.column_stats(k, None)
    q8, qs, qsum = torch_ops.quantize_qk_blocks(q, 128)
    k8, ks, ksum = torch_ops.quantize_qk_blocks(k, 64, mean=k_mean)
    ref_q8, ref_qs, ref_qsum = ops.quant_qk_blocks(q, 128, summary_dtype=torch.float64)
    assert torch.equal(q8, ref_q8) and torch.equal(qs, ref_qs) and torch.equal(qsum, ref_qsum)
    carrier, v_scale = torch_ops.prepare_v(v)
    ref_carrier, ref_v_scale = ops.quant_v_fp8(v)
    assert torch.equal(carrier.view(torch.uint8), ref_carrier.view(torch.uint8)) and torch.equal(v_scale, ref_v_scale)
    q_tiles, kv_tiles = qsum.shape[2], ksum.shape[2]
    route = torch_ops.route(qsum, ksum, q_start=2, q_stop=q_tiles, kv_start=4, kv_stop=kv_tiles, retained=5)
    assert torch.equal(route, ops.route_topk(qsum, ksum, q_start=2, q_stop=q_tiles, kv_start=4, kv_stop=kv_tiles,
                                             retained=5))
    out = torch_ops.sparse_attention(q8, k8, carrier, route, qs, ks, v_scale, q_start=2, q_stop=q_tiles)
    ref = ops.sparse_attention(q8, k8, carrier, qs, ks, v_scale, route, q_start=2, q_stop=q_tiles)
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16 and torch.equal(out, ref.contiguous())
