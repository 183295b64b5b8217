"""The torch.library operators: namespace, schemas and fake implementations
(host only; the CUDA implementations are exercised by the GPU tests)."""

import re
from pathlib import Path

import torch

PACKAGE = Path(__file__).resolve().parents[1] / "h3_optimizations_b200"


def test_every_custom_op_uses_the_pack_namespace():
    # same rule as the reference's tests/test_source_isolation.py:31-40
    declarations = []
    for path in PACKAGE.rglob("*.py"):
        text = path.read_text(encoding="utf-8")
        for match in re.finditer(r"custom_op\(", text):
            declarations.append(text[match.start():match.start() + 200])
    assert declarations
    for declaration in declarations:
        assert 'NAMESPACE + "::b200_' in declaration
    from h3_optimizations_b200 import torch_ops

    assert torch_ops.NAMESPACE == "h3_optimizations"
    for name in ("b200_quantize_qk_blocks", "b200_prepare_v", "b200_route", "b200_sparse_attention"):
        assert hasattr(torch.ops.h3_optimizations, name)


def test_fake_implementations_give_the_carrier_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode

    from h3_optimizations_b200 import torch_ops

    heads, sequence = 3, 1000
    with FakeTensorMode():
        x = torch.empty((1, heads, sequence, 128), dtype=torch.bfloat16, device="cuda")
        q8, qs, qsum = torch_ops.quantize_qk_blocks(x, 128)
        k8, ks, ksum = torch_ops.quantize_qk_blocks(x, 64, mean=torch.empty((1, heads, 128), device="cuda"))
        assert q8.dtype == torch.int8 and tuple(q8.shape) == (1, heads, sequence, 128)
        assert tuple(qs.shape) == (1, heads, 8) and tuple(ks.shape) == (1, heads, 16)
        assert tuple(qsum.shape) == (1, heads, 8, 128) and ksum.dtype == torch.float64
        carrier, v_scale = torch_ops.prepare_v(x)
        assert carrier.dtype == torch.float8_e4m3fn and tuple(carrier.shape) == (1, heads, 128, 1024)
        assert tuple(v_scale.shape) == (1, heads, 128) and v_scale.dtype == torch.float32
        route = torch_ops.route(qsum, ksum, q_start=2, q_stop=8, kv_start=4, kv_stop=16, retained=5)
        assert route.dtype == torch.int32 and tuple(route.shape) == (1, heads, 6, 4 + 5)
        out = torch_ops.sparse_attention(q8, k8, carrier, route, qs, ks, v_scale, q_start=2, q_stop=8,
                                         output_dtype=torch.float16)
        assert out.dtype == torch.float16 and tuple(out.shape) == (1, heads, sequence, 128)
