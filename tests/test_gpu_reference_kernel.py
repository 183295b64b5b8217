"""The attention kernel against the reference's own INT8 sparse kernel.  Needs a B200.

The reference pack ships one executable statement of block-sparse INT8
attention: the Triton kernels of attention/sparse/triton_sparse_kernels.py
(`_dense_kernel`, `_sparse_kernel`, launched by `launch_int8_sparse`, lines
206-246).  They import nothing but torch and Triton, so the unmodified file -
staged under oracle/_ref by oracle/build_ref.py - runs on the same GPU, on the
same seeded inputs, the same INT8 Q/K codes and the same route as
`sparse_attn_tc_kernel`.  The two differ only where the formats differ: the
reference carries V as per-(64-key block, channel) INT8 with unsigned 8-bit
probabilities (triton_sparse_kernels.py:34-42), this library carries V as
per-channel FP8-E4M3 with two E4M3 probability terms.

Both outputs are also compared with the reference's FP32 attention on the same
block mask (benchmarks/bench_sparse_backends.py:302-326), run from the staged
reference on the host.
"""

from types import SimpleNamespace

import pytest
import torch

from h3_optimizations_b200 import workloads
from oracle import h3_oracle as oracle
from oracle import ref_bridge

pytestmark = pytest.mark.gpu


def pack_v_int8_blocks(v, block=64):
    """INT8 V for the reference kernel: one scale per (key block, channel),
    ``scale = amax/127 + 1e-7``, codes rounded half away from zero, plus the
    per-block column sums of the codes (the kernel adds ``128 * sum`` back
    after its offset-by-128 probabilities).  Restates
    attention/sparse/triton_qkv_fast.py:368-393 for a scale group of one
    channel, vectorised over blocks."""
    batch, heads, sequence, dim = v.shape
    blocks = -(-sequence // block)
    padded = torch.zeros((batch, heads, blocks * block, dim), dtype=torch.float32, device=v.device)
    padded[:, :, :sequence] = v.float()
    tiles = padded.view(batch, heads, blocks, block, dim)
    scale = tiles.abs().amax(dim=3) / 127.0 + 1e-7                      # (B,H,blocks,D)
    scaled = tiles / scale[:, :, :, None, :]
    codes = (scaled + torch.where(scaled >= 0, 0.5, -0.5)).to(torch.int8)  # C-style truncation
    sums = codes.to(torch.int32).sum(dim=3)                              # (B,H,blocks,D)
    codes = codes.view(batch, heads, blocks * block, dim)[:, :, :sequence].contiguous()
    return codes, scale.contiguous(), sums.contiguous()


def run_reference_kernel(sparse, v, geo):
    """`launch_int8_sparse` of the staged reference on this library's Q/K
    carriers and route, V packed the reference's way."""
    kernels = ref_bridge.triton_kernels_module()
    v_int8, v_scale, v_sum = pack_v_int8_blocks(v)
    heads, sequence = sparse.heads, sparse.sequence
    routed = sparse.route.indices is not None
    prepared = SimpleNamespace(
        q_int8=sparse.q_int8, k_int8=sparse.k_int8, v_int8=v_int8,
        q_scale=sparse.q_scale, k_scale=sparse.k_scale, v_scale=v_scale, v_sum=v_sum,
        kv_indices=sparse.route.indices if routed else None,
        sequence=sequence, heads=heads, kv_tiles=geo.kv_tiles,
        dense_q_tiles=geo.pure_video_q_start if routed else geo.q_tiles,
        sparse_q_tiles=geo.pure_video_q_tiles if routed else 0,
        sparse_selected=sparse.route.route_len,
    )
    spec = SimpleNamespace(q_tile=128, kv_tile=64, head_dim=128, v_scale_group_size=1)
    out = torch.empty((1, heads, sequence, 128), dtype=torch.bfloat16, device=v.device)
    kernels.launch_int8_sparse(prepared, spec, out)
    torch.cuda.synchronize()
    return out


def float_reference(q, k, v, video_start, budget, route):
    """The staged reference's router + FP32 attention on the host; also checks
    that its mask is the one the GPU routed with."""
    sequence = q.shape[2]
    lut, valid, _ = ref_bridge.build_lut(q.float(), k.float(), sequence, video_start, budget)
    absolute = ref_bridge.bench_module().absolute_lut(torch, lut)
    geo = oracle.geometry(sequence, video_start)
    if route is not None:
        rows = absolute[0, :, geo.pure_video_q_start:, :route.shape[-1]]
        assert torch.equal(rows, route[0].cpu()), "GPU route differs from the reference router's"
    return ref_bridge.sparse_float_reference(q.float(), k.float(), v.float(), lut, valid)


CASES = [
    # name, spec factory, video_start, seed
    ("1024 tokens, 2 heads, gaussian", lambda: workloads.small_spec("ref", 2, 192, 832), 192, "gaussian"),
    ("benchmark layer, head 5 of 24", lambda: workloads.CONFIG1, 512, "structured"),
]


@pytest.mark.parametrize("name,make_spec,video_start,kind", CASES, ids=[c[0] for c in CASES])
def test_matches_the_reference_int8_kernel(native_lib, name, make_spec, video_start, kind):
    if not ref_bridge.available():
        pytest.skip("oracle/_ref is not staged (python oracle/build_ref.py --reference <checkout>)")
    pytest.importorskip("triton")
    from h3_optimizations_b200 import B200SparseBackend, HybridSparseConfig, runtime_options

    spec = make_spec()
    if kind == "gaussian":
        q, k, v = workloads.gaussian_qkv(spec, seed=11)
    else:
        import dataclasses

        q, k, v = workloads.structured_qkv(spec, seed=0, heads=[5])
        spec = dataclasses.replace(spec, heads=1)
    backend = B200SparseBackend(HybridSparseConfig(video_budget=0.3))
    options = runtime_options(spec.layout())
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    prepared = backend.prepare(qd, kd, vd, layer_index=0, transformer_options=options)
    ours = backend.execute(prepared)
    torch.cuda.synchronize()
    sparse = prepared.sparse
    geo = sparse.route.geometry
    theirs = run_reference_kernel(sparse, vd, geo)

    between = oracle.compare(ours.float().cpu(), theirs.float().cpu())
    flt = float_reference(q, k, v, video_start, 0.3, sparse.route.indices)
    ours_err = oracle.compare(ours.float().cpu(), flt)
    theirs_err = oracle.compare(theirs.float().cpu(), flt)
    print("\n%s\n  this kernel vs reference INT8 kernel: %s\n  this kernel vs FP32 reference:       %s\n"
          "  reference INT8 kernel vs FP32 ref:    %s" % (name, between, ours_err, theirs_err))
    assert between["cosine"] >= 0.999, between
    # Against FP32 attention both kernels are dominated by what their formats lose: the INT8
    # Q/K quantisation they share, and for this kernel the 3-bit mantissa of FP8 V (the
    # reference kernel's INT8 V with one scale per 64-key block and channel is finer).  The
    # kernel itself must add nothing to its formats: its error is held to that of the CPU
    # restatement of the same INT8-QK / FP8-V arithmetic with FP32 probabilities.
    q8, qs = oracle.quantize_blocks(q, 128)
    k8, ks = oracle.quantize_blocks(k, 64, subtract_mean=True)
    vc, vs = oracle.v_fp8_carrier(v)
    ogeo = oracle.geometry(spec.sequence, video_start)
    route = None if sparse.route.indices is None else sparse.route.indices.cpu()
    formats = oracle.sparse_attention_int8_fp8(q8, qs, k8, ks, vc, vs, ogeo, route)
    formats_err = oracle.compare(formats, flt)
    print("  INT8-QK / FP8-V formats (CPU, FP32 P) vs FP32 reference: %s" % formats_err)
    assert ours_err["rel_rmse"] <= 1.05 * formats_err["rel_rmse"], (ours_err, formats_err)
    assert ours_err["cosine"] >= theirs_err["cosine"] - 5e-4, (ours_err, theirs_err)
    gate = oracle.compare(ours.float().cpu(), formats)
    assert gate["cosine"] >= 0.999 and gate["rel_max_abs"] <= 2e-2, gate
