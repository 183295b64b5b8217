"""Backend / projector protocol on the device.  Needs a B200."""

import pytest
import torch

from h3_optimizations_b200 import workloads
from oracle import h3_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend(native_lib):
    from h3_optimizations_b200 import B200SparseBackend, HybridSparseConfig

    return B200SparseBackend(
        HybridSparseConfig(video_budget=0.3, early_steps=2, early_kv=0.5, late_steps=2, late_kv=0.5)
    )


def test_step_schedule_drives_the_route(backend):
    from h3_optimizations_b200 import runtime_options

    spec = workloads.small_spec("b", 2, 256, 1024)
    q, k, v = (t.cuda() for t in workloads.gaussian_qkv(spec, seed=4))
    expected = {-1: 0.3, 0: 0.5, 1: 0.5, 2: 0.3, 27: 0.3, 28: 0.5, 29: 0.5}
    for step, budget in expected.items():
        prepared = backend.prepare(q, k, v, layer_index=0,
                                   transformer_options=runtime_options(spec.layout(), step, 30))
        meta = prepared.sparse.metadata
        assert meta["requested_video_budget"] == budget
        assert meta["retained_video_kv_tiles"] == {0.3: 5, 0.5: 8}[budget]
        out = backend.execute(prepared)
        assert out.dtype == torch.bfloat16 and tuple(out.shape) == (1, 2, 1280, 128)
    torch.cuda.synchronize()


def test_prepare_projected_uses_supplied_carriers(backend):
    from h3_optimizations_b200 import PreparedFusedQKV, runtime_options

    spec = workloads.small_spec("b", 2, 128, 512)
    q, k, v = workloads.gaussian_qkv(spec, seed=6)
    q8, qs = oracle.quantize_blocks(q, 128)
    k8, ks = oracle.quantize_blocks(k, 64)
    projected = PreparedFusedQKV(
        q_int8=q8.cuda(), q_scale=qs.cuda(), k_int8=k8.cuda(), k_scale=ks.cuda(), v=v.cuda(),
        q_summary=oracle.block_summaries(q, 128, torch.float32).cuda(),
        k_summary=oracle.block_summaries(k, 64, torch.float32).cuda(),
        output_dtype=torch.bfloat16, sequence=640, heads=2, head_dim=128, layer_index=3, smooth_k=False,
    )
    options = runtime_options(spec.layout())
    prepared = backend.prepare_projected(projected, layer_index=3, transformer_options=options)
    assert prepared.sparse.q_int8.data_ptr() == projected.q_int8.data_ptr()  # no repack
    assert prepared.sparse.metadata["qkv_projection"] == "fused_int8"
    out = backend.execute(prepared).float().cpu()
    geo = oracle.geometry(640, 128)
    retained = oracle.retained_tiles(0.3, geo)
    selected = oracle.select_tiles(projected.q_summary.cpu(), projected.k_summary.cpu(), geo, retained)
    route = oracle.compact_route(selected, geo)
    assert torch.equal(prepared.sparse.route.indices.cpu(), route)
    vc, vs = oracle.v_fp8_carrier(v)
    ref = oracle.sparse_attention_int8_fp8(q8, qs, k8, ks, vc, vs, geo, route)
    m = oracle.compare(out, ref)
    assert m["cosine"] >= 0.999 and m["rel_max_abs"] <= 2e-2, m


def test_contract_errors(backend):
    from h3_optimizations_b200 import SparseSageError, runtime_options

    spec = workloads.small_spec("b", 1, 128, 256)
    q, k, v = (t.cuda() for t in workloads.gaussian_qkv(spec, seed=1))
    with pytest.raises(SparseSageError, match="runtime snapshot"):
        backend.prepare(q, k, v, layer_index=0, transformer_options={})
    other = workloads.small_spec("b", 1, 128, 512)
    with pytest.raises(SparseSageError, match="does not match attention sequence"):
        backend.prepare(q, k, v, layer_index=0, transformer_options=runtime_options(other.layout()))
    with pytest.raises(SparseSageError, match="batch 1"):
        backend.prepare(q.repeat(2, 1, 1, 1), k.repeat(2, 1, 1, 1), v.repeat(2, 1, 1, 1), layer_index=0,
                        transformer_options=runtime_options(spec.layout()))
    with pytest.raises(SparseSageError, match="requires CUDA"):
        backend.prepare(q.cpu(), k.cpu(), v.cpu(), layer_index=0,
                        transformer_options=runtime_options(spec.layout()))
    assert backend.as_status()["sparse_architecture"] == "sm_100a"
    assert backend.installation_signature == backend.installation_signature


def test_forward_host_matches_device_path(backend):
    """The pipelined host entry (head chunks over three streams) returns what
    prepare + execute return on device-resident tensors: heads are independent,
    so chunking changes nothing, including a ragged last chunk and slot reuse."""
    from h3_optimizations_b200 import runtime_options

    spec = workloads.small_spec("host", 7, 256, 1024)
    q, k, v = workloads.gaussian_qkv(spec, seed=9)
    options = runtime_options(spec.layout(), 5, 30)
    prepared = backend.prepare(q.cuda(), k.cuda(), v.cuda(), layer_index=0, transformer_options=options)
    expected = backend.execute(prepared).contiguous().cpu()
    qh, kh, vh = (t.contiguous().pin_memory() for t in (q, k, v))
    for chunk in (2, 3, 7):
        out = backend.forward_host(qh, kh, vh, layer_index=0, transformer_options=options, heads_per_chunk=chunk)
        torch.cuda.synchronize()
        assert out.is_pinned() and tuple(out.shape) == tuple(q.shape)
        assert torch.equal(out, expected), "heads_per_chunk=%d" % chunk
    # a second call reuses the staging slots and streams
    again = backend.forward_host(qh, kh, vh, layer_index=0, transformer_options=options, heads_per_chunk=2)
    torch.cuda.synchronize()
    assert torch.equal(again, expected)
    with pytest.raises(Exception, match="host tensors"):
        backend.forward_host(q.cuda(), k.cuda(), v.cuda(), layer_index=0, transformer_options=options)


def test_captured_layer_call_replays_every_kernel(backend):
    """``backend.capture``: prepare + execute as one CUDA graph.  A replay must give
    the eager result bit for bit, follow the contents of the input tensors (all the
    kernels run again, nothing is cached), and leave the eager path usable."""
    from h3_optimizations_b200 import runtime_options

    spec = workloads.small_spec("graph", 2, 192, 832 + 17)
    q, k, v = (t.cuda() for t in workloads.gaussian_qkv(spec, seed=9))
    options = runtime_options(spec.layout(), 5, 30)

    def eager():
        return backend.execute(backend.prepare(q, k, v, layer_index=0, transformer_options=options))

    first = eager().clone()
    captured = backend.capture(q, k, v, layer_index=0, transformer_options=options)
    assert torch.equal(captured.replay(), first)
    # new contents in the same buffers: the replay recomputes statistics, carriers, route and output
    q2, k2, v2 = (t.cuda() for t in workloads.gaussian_qkv(spec, seed=10))
    q.copy_(q2); k.copy_(k2); v.copy_(v2)
    second = captured.replay().clone()
    torch.cuda.synchronize()
    assert not torch.equal(second, first)
    assert torch.equal(eager(), second)
    backend.check_status()
