"""Chunked ConvRot INT8 QKV projection against the oracle.  Needs a B200.

The rotation is unpinned in the reference (it lives in comfy_kitchen); it is
pinned here by the oracle's FWHT with the same stage order (bit-exact codes)
and by the invariance test in tests/test_oracle_golden.py.  The integer GEMM is
exact, so the bf16 staging must match the oracle bit for bit."""

from types import SimpleNamespace

import pytest
import torch

from h3_optimizations_b200 import workloads
from oracle import h3_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(native_lib):
    from h3_optimizations_b200 import ops as module

    return module


@pytest.mark.parametrize("rows,hidden", [(1, 256), (37, 512), (300, 3072), (4096, 3072)])
def test_convrot_rows_are_bit_exact(ops, rows, hidden):
    gen = torch.Generator().manual_seed(rows)
    x = (torch.randn((rows, hidden), generator=gen) * 1.7).to(torch.bfloat16)
    x[0, :] = 0 if rows > 1 else x[0, :]  # an all-zero row takes scale 1
    codes, scale = ops.convrot_quant_rows(x.cuda())
    ref_codes, ref_scale = oracle.convrot_quantize_rows(x)
    assert torch.equal(scale.cpu(), ref_scale)
    assert torch.equal(codes.cpu(), ref_codes)


@pytest.mark.parametrize("rows,heads", [(128, 1), (300, 2), (1000, 3), (4096, 2)])
def test_gemm_chunk_matches_exact_integer_gemm(ops, rows, heads):
    hidden = 1024
    x, w, w_scale = workloads.projection_inputs(rows, hidden=hidden, heads=heads, seed=rows)
    x_i8, x_scale = oracle.convrot_quantize_rows(x)
    ref = oracle.qkv_project_int8(x_i8, x_scale, w, w_scale)          # (rows, 3*H*128) bf16
    staging = torch.full((3 * heads, rows + 64, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.qkv_gemm_chunk(x_i8.cuda(), x_scale.cuda(), w.cuda(), w_scale.cuda(), staging, row_start=64, status=status)
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    got = staging[:, 64:].permute(1, 0, 2).reshape(rows, 3 * heads * 128).cpu()
    assert torch.equal(got.view(torch.int16), ref.view(torch.int16))
    assert bool(torch.isnan(staging[:, :64].float()).all()), "rows before the chunk must stay untouched"


@pytest.mark.parametrize("smooth_k", [True, False])
def test_projector_builds_the_same_carriers_as_the_oracle(ops, smooth_k):
    from h3_optimizations_b200 import ChunkedSparseQKVProjector

    sequence, hidden, heads = 700, 768, 2
    x, w, w_scale = workloads.projection_inputs(sequence, hidden=hidden, heads=heads, seed=3)
    module = SimpleNamespace(heads=heads, head_dim=128, qkv_weight_int8=w.cuda(), qkv_weight_scale=w_scale.cuda())
    projector = ChunkedSparseQKVProjector(chunk_rows=256, smooth_k=smooth_k)
    prepared = projector.project(module, x.cuda(), None, layer_index=5, transformer_options={})
    torch.cuda.synchronize()
    assert projector.try_project(module, x.cuda(), torch.zeros(1), layer_index=5, transformer_options={}) is None

    x_i8, x_scale = oracle.convrot_quantize_rows(x)
    y = oracle.qkv_project_int8(x_i8, x_scale, w, w_scale)
    q, k, v = oracle.split_heads_hnd(y, heads)
    q8, qs = oracle.quantize_blocks(q, 128)
    assert torch.equal(prepared.q_int8.cpu(), q8) and torch.equal(prepared.q_scale.cpu(), qs)
    if smooth_k:
        # the device mean is an FP64 sum rounded once; hand the same mean to the oracle
        k_mean, _ = ops.column_stats(k.cuda().contiguous(), None)
        k8, ks = oracle.quantize_blocks(k, 64, mean=k_mean.cpu())
    else:
        k8, ks = oracle.quantize_blocks(k, 64)
    assert torch.equal(prepared.k_int8.cpu(), k8) and torch.equal(prepared.k_scale.cpu(), ks)
    vc, vs = oracle.v_fp8_carrier(v)
    assert torch.equal(prepared.v_scale.cpu(), vs)
    assert torch.equal(prepared.v_carrier.cpu().view(torch.uint8), vc.view(torch.uint8))
    assert torch.allclose(prepared.q_summary.cpu(), oracle.block_summaries(q, 128, torch.float32), atol=1e-5)
    assert torch.allclose(prepared.k_summary.cpu(), oracle.block_summaries(k, 64, torch.float32), atol=1e-5)
    assert prepared.smooth_k == smooth_k and prepared.layer_index == 5 and prepared.v is None


def test_projection_feeds_the_backend_end_to_end(ops):
    """config-2 shape in miniature: projection -> prepare_projected -> execute,
    checked against the oracle run on the oracle's own projection."""
    from h3_optimizations_b200 import B200SparseBackend, ChunkedSparseQKVProjector, HybridSparseConfig, runtime_options

    spec = workloads.small_spec("p", 2, 256, 1024)
    sequence, hidden, heads = spec.sequence, 512, 2
    x, w, w_scale = workloads.projection_inputs(sequence, hidden=hidden, heads=heads, seed=8)
    module = SimpleNamespace(heads=heads, head_dim=128, qkv_weight_int8=w.cuda(), qkv_weight_scale=w_scale.cuda())
    backend = B200SparseBackend(HybridSparseConfig(mode="sage128_fused_qkv", video_budget=0.3))
    assert isinstance(backend.projector, ChunkedSparseQKVProjector) and backend.projector.chunk_rows == 4096
    projected = ChunkedSparseQKVProjector(chunk_rows=512).project(module, x.cuda(), None, layer_index=0,
                                                                  transformer_options={})
    prepared = backend.prepare_projected(projected, layer_index=0, transformer_options=runtime_options(spec.layout()))
    out = backend.execute(prepared).float().cpu()

    x_i8, x_scale = oracle.convrot_quantize_rows(x)
    q, k, v = oracle.split_heads_hnd(oracle.qkv_project_int8(x_i8, x_scale, w, w_scale), heads)
    geo, retained, selected, route = oracle.build_route(q.float(), k.float(), sequence, 256, 0.3)
    assert torch.equal(prepared.sparse.route.indices.cpu(), route)
    q8, qs = oracle.quantize_blocks(q, 128)
    k8, ks = oracle.quantize_blocks(k, 64, subtract_mean=True)
    vc, vs = oracle.v_fp8_carrier(v)
    ref = oracle.sparse_attention_int8_fp8(q8, qs, k8, ks, vc, vs, geo, route)
    m = oracle.compare(out, ref)
    assert m["cosine"] >= 0.999 and m["rel_max_abs"] <= 2e-2, m


def test_projection_errors(ops):
    from h3_optimizations_b200 import ChunkedSparseQKVProjector, FusedQKVError
    from h3_optimizations_b200.projector import run_chunked_sparse_qkv

    with pytest.raises(FusedQKVError, match="multiple of 128"):
        ChunkedSparseQKVProjector(chunk_rows=192)
    x = torch.zeros((256, 512), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((384, 512), dtype=torch.int8, device="cuda")
    s = torch.ones((384,), dtype=torch.float32, device="cuda")
    with pytest.raises(FusedQKVError, match="rank-2 CUDA BF16"):
        run_chunked_sparse_qkv(x.float(), w, s, heads=1)
    with pytest.raises(FusedQKVError, match="QKV weight must be int8"):
        run_chunked_sparse_qkv(x, w, s, heads=2)
    module = SimpleNamespace(heads=1, head_dim=128)
    with pytest.raises(FusedQKVError, match="does not expose"):
        ChunkedSparseQKVProjector().project(module, x, None, layer_index=0, transformer_options={})


@pytest.mark.parametrize("rope_dtype", [None, torch.bfloat16, torch.float32])
def test_gemm_epilogue_norm_and_rope_are_bit_exact(ops, rope_dtype):
    """Per-head RMS norm (+ split-half rotation) of the Q and K heads inside the
    GEMM epilogue against the oracle's restatement of the reference epilogue;
    V heads must come out exactly as without it.  The chunk starts at row 128 of
    a longer sequence, so the rotation has to pick the chunk's own rows."""
    rows, hidden, heads, sequence, start = 300, 512, 2, 512, 128
    x, w, w_scale = workloads.projection_inputs(rows, hidden=hidden, heads=heads, seed=11)
    x_i8, x_scale = oracle.convrot_quantize_rows(x)
    gen = torch.Generator().manual_seed(5)
    q_norm = torch.rand(128, generator=gen) + 0.5
    k_norm = torch.rand(128, generator=gen) + 0.5
    rope = None if rope_dtype is None else oracle.make_rope(sequence).to(rope_dtype)
    y = oracle.qkv_project_int8(x_i8, x_scale, w, w_scale)
    ref = oracle.rms_norm_rope_split_half(y, heads, q_norm, k_norm, 1e-6,
                                          None if rope is None else rope[:, start:start + rows])
    staging = torch.full((3 * heads, sequence, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.qkv_gemm_chunk(x_i8.cuda(), x_scale.cuda(), w.cuda(), w_scale.cuda(), staging, row_start=start, status=status,
                       q_norm=q_norm.cuda(), k_norm=k_norm.cuda(), epsilon=1e-6,
                       rope=None if rope is None else rope.cuda())
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    got = staging[:, start:start + rows].permute(1, 0, 2).reshape(rows, 3 * heads * 128).cpu()
    assert torch.equal(got.view(torch.int16), ref.view(torch.int16))
    assert torch.equal(got[:, 2 * heads * 128:].view(torch.int16), y[:, 2 * heads * 128:].view(torch.int16))
    assert bool(torch.isnan(staging[:, :start].float()).all()) and bool(torch.isnan(staging[:, start + rows:].float()).all())
    with pytest.raises(Exception, match="go together"):
        ops.qkv_gemm_chunk(x_i8.cuda(), x_scale.cuda(), w.cuda(), w_scale.cuda(), staging, q_norm=q_norm.cuda())


def test_projector_applies_the_modules_norm_and_rope(ops):
    """A module with q_norm / k_norm and a rotary table goes through the chunked
    provider (it no longer declines), and the carriers are the oracle's carriers
    of the normed and rotated projection; the forward transaction built on it
    returns out_proj(attention)."""
    from h3_optimizations_b200 import B200SparseBackend, ChunkedSparseQKVProjector, HybridSparseConfig, runtime_options
    from h3_optimizations_b200.attention_forward import make_forward

    spec = workloads.small_spec("rope", 2, 256, 1024)
    sequence, hidden, heads = spec.sequence, 512, 2
    x, w, w_scale = workloads.projection_inputs(sequence, hidden=hidden, heads=heads, seed=13)
    gen = torch.Generator().manual_seed(6)
    norm = lambda: SimpleNamespace(weight=(torch.rand(128, generator=gen) + 0.5).to(torch.bfloat16).cuda(), eps=1e-6)
    out_proj = torch.nn.Linear(heads * 128, hidden, bias=False).to(device="cuda", dtype=torch.bfloat16)
    module = SimpleNamespace(heads=heads, head_dim=128, qkv_weight_int8=w.cuda(), qkv_weight_scale=w_scale.cuda(),
                             q_norm=norm(), k_norm=norm(), out_proj=out_proj)
    rope = oracle.make_rope(sequence).cuda()
    projector = ChunkedSparseQKVProjector(chunk_rows=512)
    prepared = projector.try_project(module, x.cuda(), rope, layer_index=1, transformer_options={})
    assert prepared is not None

    x_i8, x_scale = oracle.convrot_quantize_rows(x)
    y = oracle.rms_norm_rope_split_half(oracle.qkv_project_int8(x_i8, x_scale, w, w_scale), heads,
                                        module.q_norm.weight.cpu(), module.k_norm.weight.cpu(), 1e-6, rope.cpu())
    q, k, v = oracle.split_heads_hnd(y, heads)
    q8, qs = oracle.quantize_blocks(q, 128)
    assert torch.equal(prepared.q_int8.cpu(), q8) and torch.equal(prepared.q_scale.cpu(), qs)
    k_mean, _ = ops.column_stats(k.cuda().contiguous(), None)
    k8, ks = oracle.quantize_blocks(k, 64, mean=k_mean.cpu())
    assert torch.equal(prepared.k_int8.cpu(), k8) and torch.equal(prepared.k_scale.cpu(), ks)
    vc, vs = oracle.v_fp8_carrier(v)
    assert torch.equal(prepared.v_carrier.cpu().view(torch.uint8), vc.view(torch.uint8))

    backend = B200SparseBackend(HybridSparseConfig(video_budget=0.3))
    options = runtime_options(spec.layout())
    with torch.no_grad():
        got = make_forward(module, 1, backend=backend, projector=projector)(x.cuda(), rope, options)
        attention = backend.execute(backend.prepare_projected(prepared, layer_index=1, transformer_options=options))
        expected = out_proj(attention.transpose(1, 2).reshape(sequence, heads * 128))
    assert tuple(got.shape) == (sequence, hidden) and torch.equal(got, expected)
    with pytest.raises(Exception, match="needs the module's q_norm"):
        projector.project(SimpleNamespace(heads=heads, head_dim=128, qkv_weight_int8=w.cuda(),
                                          qkv_weight_scale=w_scale.cuda()), x.cuda(), rope, layer_index=0,
                          transformer_options={})
