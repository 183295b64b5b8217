"""A device-side wait that runs out.  Needs a B200.

Every mbarrier wait of the attention kernel is bounded.  This test makes one
run out on purpose, the safe way: a one-CTA launch with the self-test flag
``H3S_ATTN_TEST_DROP_KV_LOAD`` (the producer never issues the first K/V load)
and a 1 ms budget.  Nothing faults and nothing spins forever: the wait gives
up, the kernel records which wait it was, releases its tensor memory and
returns, and the next launch on the same context runs normally."""

import pytest
import torch

from h3_optimizations_b200 import workloads

pytestmark = pytest.mark.gpu

K_V_TILE_LOAD = 2  # status code of the wait for a K/V tile


@pytest.fixture()
def short_budget(native_lib):
    from h3_optimizations_b200 import ops

    previous = ops.set_wait_budget_ns(1_000_000)  # 1 ms (4 ms for the waits furthest down the pipeline)
    yield ops
    ops.set_wait_budget_ns(previous)


def _carriers(ops):
    spec = workloads.small_spec("wait", 1, 64, 64)  # 128 tokens: one query tile, two KV tiles, one CTA
    q, k, v = (t.cuda() for t in workloads.gaussian_qkv(spec, seed=5))
    k_mean, v_scale = ops.column_stats(k, v)
    q8, qs, _ = ops.quant_qk_blocks(q, 128)
    k8, ks, _ = ops.quant_qk_blocks(k, 64, mean=k_mean)
    vc, _ = ops.quant_v_fp8(v, v_scale)
    return q8, k8, vc, qs, ks, v_scale


def test_expired_wait_reports_and_leaves_the_device_usable(short_budget):
    ops = short_budget
    args = _carriers(ops)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    good = ops.sparse_attention(*args, out_dtype=torch.float32, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    ops.sparse_attention(*args, out_dtype=torch.float32, status=status, extra_flags=ops.ATTN_TEST_DROP_KV_LOAD)
    stop.record()
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    code, cta, head, tile = status.tolist()
    assert code == K_V_TILE_LOAD, "the wait for the K/V tile must be the one that reports, got %d" % code
    assert (cta, head, tile) == (0, 0, 0)
    assert start.elapsed_time(stop) < 50.0, "the launch must end a few budgets after it started"

    status.zero_()
    again = ops.sparse_attention(*args, out_dtype=torch.float32, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    assert torch.equal(again, good), "tensor memory was released: the next launch is unaffected"


def test_backend_surfaces_the_status(short_budget):
    from h3_optimizations_b200 import B200SparseBackend, HybridSparseConfig
    from h3_optimizations_b200.errors import SparseSageError

    ops = short_budget
    args = _carriers(ops)
    backend = B200SparseBackend(HybridSparseConfig(video_budget=0.3))
    word = backend._status_slot(torch.device("cuda", torch.cuda.current_device()))[0]
    ops.sparse_attention(*args, out_dtype=torch.float32, status=word, extra_flags=ops.ATTN_TEST_DROP_KV_LOAD)
    with pytest.raises(SparseSageError, match="K/V tile load"):
        backend.check_status()
    backend.check_status()  # the word was cleared
