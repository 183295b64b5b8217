"""Router kernel: the block mask must equal the reference router's bit for bit
(fixtures produced by the reference on FP32 inputs).  Needs a B200."""

import json

import numpy as np
import pytest
import torch

from h3_optimizations_b200 import workloads
from oracle import h3_oracle as oracle
from tests.helpers import checksum, layout_of, mask_from_bits, mask_from_route

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def router(native_lib):
    from h3_optimizations_b200.router import SparseTileRouter

    return SparseTileRouter()


def _inputs(name):
    if name == "s350":
        q, k, _ = workloads.gaussian_qkv(workloads.small_spec("r350", 2, 96, 254), seed=11, widen=True)
    elif name == "s1024":
        q, k, _ = workloads.structured_qkv(workloads.small_spec("r1024", 3, 256, 768), seed=5)
    elif name == "config0":
        q, k, _ = workloads.gaussian_qkv(workloads.CONFIG0, seed=0, widen=True)
    else:
        q, k, _ = workloads.structured_qkv(workloads.CONFIG1, seed=0)
    return q, k


@pytest.mark.parametrize("name", ["s350", "s1024", "config0", "config1"])
def test_mask_is_bit_exact_against_reference_router(router, golden_dir, name):
    data = np.load(golden_dir / ("router_%s.npz" % name))
    q, k = _inputs(name)
    sequence, video_start, budget = int(data["sequence"]), int(data["video_start"]), float(data["budget"])
    layout = layout_of(sequence, video_start)
    # bf16 inputs hold the same values as the FP32-widened tensors the reference saw
    route = router.build_route(q.cuda(), k.cuda(), layout, budget)
    geo = route.geometry
    assert route.metadata.as_dict() == json.loads(str(data["meta"]))
    got = mask_from_route(route.indices, geo, q.shape[1])
    if checksum(q.float(), k.float()) == str(data["input_sha"]):
        expected = mask_from_bits(data["mask_bits"], geo.kv_tiles)
    else:  # this platform's RNG differs from the fixture's: compare with the oracle run here
        ogeo, _, _, oroute = oracle.build_route(q.float(), k.float(), sequence, video_start, budget)
        expected = mask_from_route(oroute, ogeo, q.shape[1])
    differing = int((got != expected).any(dim=-1).sum())
    assert differing == 0, "%d of %d rows differ" % (differing, got.shape[0] * got.shape[1])
    rows = route.indices[0].cpu()
    assert bool((rows[..., 1:] > rows[..., :-1]).all()), "route rows must be strictly ascending"
    lut, valid, _ = router.build_lut(q.cuda(), k.cuda(), layout, budget)
    assert np.array_equal(valid.cpu().numpy(), data["valid"])
    if "lut" in data and checksum(q.float(), k.float()) == str(data["input_sha"]):
        assert torch.equal(lut.cpu(), torch.from_numpy(data["lut"]))


def test_summaries_entry_matches_reference_compact_route(router, golden_dir):
    data = np.load(golden_dir / "router_summaries512.npz")
    qs, ks = torch.from_numpy(data["q_summary"]).cuda(), torch.from_numpy(data["k_summary"]).cuda()
    layout = layout_of(512, 192)
    route = router.build_route_from_summaries(qs, ks, layout, 0.3)
    assert torch.equal(route.indices.cpu(), torch.from_numpy(data["route"]))
    lut, valid, _ = router.build_lut_from_summaries(qs, ks, layout, 0.3)
    assert torch.equal(lut.cpu(), torch.from_numpy(data["lut"]))
    assert torch.equal(valid.cpu(), torch.from_numpy(data["valid"]))
    for dtype in (torch.float64, torch.bfloat16):  # other summary types select on their own values
        r = router.build_route_from_summaries(qs.to(dtype), ks.to(dtype), layout, 0.3)
        geo = r.geometry
        sel = oracle.select_tiles(qs.cpu().to(dtype).double(), ks.cpu().to(dtype).double(),
                                  oracle.geometry(512, 192), r.retained)
        assert torch.equal(r.indices.cpu(), oracle.compact_route(sel, oracle.geometry(512, 192)))
        assert geo.pure_video_kv_start == 3


def test_known_answers_full_budget_and_ties(router):
    # reference tests/test_router.py:36-101
    q = torch.zeros((1, 2, 384, 128))
    k = torch.zeros_like(q)
    q[0, 0, 128:, 0] = 1
    q[0, 1, 128:, 1] = 1
    for index, value in enumerate((4.0, 3.0, 2.0, 1.0), start=2):
        k[0, 0, index * 64:(index + 1) * 64, 0] = value
    for index, value in enumerate((1.0, 2.0, 3.0, 4.0), start=2):
        k[0, 1, index * 64:(index + 1) * 64, 1] = value
    layout = layout_of(384, 128)
    route = router.build_route(q.cuda(), k.cuda(), layout, 0.5)
    assert route.indices.cpu()[0, :, 0].tolist() == [[0, 1, 2, 3], [0, 1, 4, 5]]
    assert route.metadata.retained_video_kv_tiles == 2 and route.metadata.actual_video_tile_density == 0.5
    # full budget: dense, nothing launched (tests/test_router.py:118-133)
    dense = router.build_route(q.cuda(), k.cuda(), layout, 1.0)
    assert dense.indices is None and dense.metadata.sparse_q_tiles == 0 and dense.metadata.full_mask_density == 1.0
    lut, valid, _ = router.build_lut(q.cuda(), k.cuda(), layout, 1.0)
    assert int(valid.min()) == 6 and torch.cumsum(lut, -1)[0, 0, 0].tolist() == list(range(6))
    # all-equal scores: the lower tile indices win
    zeros = torch.zeros((1, 1, 640, 128), device="cuda")
    tie = router.build_route(zeros, zeros, layout_of(640, 128), 0.3)
    assert tie.indices.cpu()[0, 0].tolist() == [[0, 1, 2, 3, 4]] * 4


def test_generalised_layout_video_first(router):
    """The benchmark description words the layout as video followed by text; the reference router rejects
    that layout, this router treats every tile outside the video range as dense."""
    from h3_optimizations_b200.errors import SparseRouterError
    from h3_optimizations_b200.router import SparseTileRouter

    spec = workloads.CONFIG0_VIDEO_FIRST
    q, k, _ = workloads.gaussian_qkv(spec, seed=0, widen=True)
    route = router.build_route(q.cuda(), k.cuda(), spec.layout(), 0.3)
    geo, retained, _, oroute = oracle.build_route(q, k, spec.sequence, 0, 0.3, video_stop=2048)
    assert route.retained == retained == 10
    assert torch.equal(route.indices.cpu(), oroute)
    assert route.indices.cpu()[0, 0, 0, -4:].tolist() == [32, 33, 34, 35]
    with pytest.raises(SparseRouterError, match="final packed segment"):
        SparseTileRouter(require_video_last=True).geometry(spec.layout())
    with pytest.raises(SparseRouterError, match="delta LUT"):
        router.build_lut(q.cuda(), k.cuda(), spec.layout(), 0.3)


def test_router_errors(router):
    from h3_optimizations_b200.errors import SparseRouterError

    q = torch.zeros((1, 1, 384, 128), device="cuda")
    with pytest.raises(SparseRouterError, match="video_budget"):
        router.build_route(q, q, layout_of(384, 128), 0.001)
    with pytest.raises(SparseRouterError, match="does not match Q/K sequence"):
        router.build_route(q, q, layout_of(512, 128), 0.5)
    with pytest.raises(SparseRouterError, match="no pure-video"):
        router.geometry(layout_of(384, 383))
