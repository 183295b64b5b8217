"""Host-side logic and the C-ABI surface; no GPU needed."""

import ctypes
import json
import re
from pathlib import Path

import pytest
import torch

from h3_optimizations_b200 import HybridSparseConfig, resolve_video_budget, workloads
from h3_optimizations_b200.errors import SparseRouterError, SparseSageError
from oracle import h3_oracle as oracle
from tests.helpers import layout_of

ROOT = Path(__file__).resolve().parents[1]


def test_library_builds_loads_and_exports_every_declared_symbol(native_lib):
    from h3_optimizations_b200 import _native

    header = (ROOT / "include" / "h3sparse.h").read_text()
    declared = set(re.findall(r"\b(h3s_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in include/h3sparse.h"
    assert declared == set(_native.PROTOTYPES), declared ^ set(_native.PROTOTYPES)
    raw = ctypes.CDLL(str(_native.LIB_PATH))
    for name in declared:
        assert hasattr(raw, name), "library does not export %s" % name
    assert native_lib.h3s_abi_version() == _native.ABI_VERSION
    assert native_lib.h3s_column_stats_scratch_bytes(24) == 24 * 128 * 12


def test_argument_validation_runs_before_any_device_work(native_lib):
    """Invalid arguments are rejected on the host, so these calls are safe
    without a GPU: nothing is launched."""
    from h3_optimizations_b200 import _native

    rc = native_lib.h3s_quant_qk_blocks(None, 1, 128, 128, None, None, None, None, 0, 1, 128, 0, 128, 32, None)
    assert rc == -1 and b"block must be 128 or 64" in native_lib.h3s_last_error()
    rc = native_lib.h3s_route_topk(None, None, 0, 1, 1, 1, 0, 1, 0, 1, 1, None, None)
    assert rc == -1 and b"NULL" in native_lib.h3s_last_error()
    rc = native_lib.h3s_sparse_attn_fwd(None, None, None, None, None, None, None, 0, 0, 0, None, 1, 0, 0, 1, 1, 0,
                                        None, None)
    assert rc == -1
    with pytest.raises(_native.NativeError, match="no CPU path"):
        from h3_optimizations_b200 import ops

        ops.quant_qk_blocks(torch.zeros((1, 1, 128, 128), dtype=torch.bfloat16), 128)


def test_missing_library_fails_loudly(tmp_path):
    from h3_optimizations_b200 import _native

    with pytest.raises(_native.NativeError, match="no CPU fallback"):
        _native.load(tmp_path / "libh3sparse.so")


def test_density_schedule_matches_reference_tables(golden_dir):
    for table in json.loads((golden_dir / "schedule.json").read_text()):
        kwargs = dict(table["config"])
        if "layer_video_budgets" in kwargs:
            kwargs["layer_video_budgets"] = tuple(kwargs["layer_video_budgets"])
        config = HybridSparseConfig(**kwargs)
        layer = 7 if config.layer_video_budgets is not None else None
        for step, expected in table["budgets"]:
            assert resolve_video_budget(config, step, table["total_steps"], layer) == expected
    # the long-sequence schedule: 30 steps, 2 early and 2 late at 50 %, the rest at 30 %
    config = HybridSparseConfig(video_budget=0.3, early_steps=2, early_kv=0.5, late_steps=2, late_kv=0.5)
    budgets = [resolve_video_budget(config, s, 30) for s in range(30)]
    assert budgets == [0.5, 0.5] + [0.3] * 26 + [0.5, 0.5]


def test_config_validation():
    with pytest.raises(ValueError, match="video_budget"):
        HybridSparseConfig(video_budget=0.001)
    with pytest.raises(ValueError, match="incomplete"):
        HybridSparseConfig(early_steps=2)
    with pytest.raises(ValueError, match="cannot be combined"):
        HybridSparseConfig(denser_early_late_steps=True, early_steps=1, early_kv=0.5, late_steps=1, late_kv=0.5)
    with pytest.raises(ValueError, match="exactly 50"):
        HybridSparseConfig(layer_video_budgets=(0.5,) * 3)
    with pytest.raises(ValueError, match="unavailable"):
        HybridSparseConfig(mode="nope")
    with pytest.raises(ValueError, match="layer_index is required"):
        resolve_video_budget(HybridSparseConfig(layer_video_budgets=(0.5,) * 50), 0, 10)
    a = HybridSparseConfig(video_budget=0.3)
    assert a.signature == HybridSparseConfig(video_budget=0.3).signature != HybridSparseConfig().signature


@pytest.mark.parametrize("spec", [workloads.CONFIG0, workloads.CONFIG1, workloads.CONFIG3, workloads.CONFIG4,
                                  workloads.CONFIG0_VIDEO_FIRST])
def test_router_geometry_and_metadata_agree_with_oracle(spec):
    from h3_optimizations_b200.router import SparseTileRouter

    router = SparseTileRouter()
    geo = router.geometry(spec.layout())
    assert router.geometry(spec.layout()) is geo  # cached by layout signature
    start, stop = spec.video_range
    ogeo = oracle.geometry(spec.sequence, start, stop)
    for name in ("sequence", "q_tiles", "kv_tiles", "pure_video_q_start", "pure_video_q_stop",
                 "pure_video_kv_start", "pure_video_kv_stop"):
        assert getattr(geo, name) == getattr(ogeo, name), name
    for budget in (0.01, 0.1, 0.3, 0.5, 0.999, 1.0):
        retained = router._retained(budget, geo)
        assert retained == oracle.retained_tiles(budget, ogeo)
        assert router._metadata(geo, budget, retained).as_dict() == oracle.mask_metadata(ogeo, budget, retained)


def test_survey_geometry_numbers():
    from h3_optimizations_b200.router import SparseTileRouter

    router = SparseTileRouter()
    g1 = router.geometry(workloads.CONFIG1.layout())
    assert (g1.q_tiles, g1.kv_tiles, g1.pure_video_q_start, g1.pure_video_kv_start) == (260, 520, 4, 8)
    assert router._retained(0.3, g1) == 154
    assert workloads.attention_pair_count(g1, 154) * 24 == 1045248
    g3 = router.geometry(workloads.CONFIG3.layout())
    assert (g3.q_tiles, g3.kv_tiles) == (595, 1190)
    assert [router._retained(b, g3) for b in (0.1, 0.3, 0.5, 1.0)] == [119, 355, 591, 1182]
    g4 = router.geometry(workloads.CONFIG4.layout())
    assert (g4.pure_video_q_start, g4.pure_video_kv_start) == (24, 48)


def test_router_and_backend_reject_bad_input_without_a_device():
    from h3_optimizations_b200.backend import B200SparseBackend
    from h3_optimizations_b200.router import SparseTileRouter

    router = SparseTileRouter()
    with pytest.raises(SparseRouterError, match="final packed segment"):
        SparseTileRouter(require_video_last=True).geometry(layout_of(2304, 0, 2048))
    with pytest.raises(SparseRouterError, match="empty"):
        router.geometry(layout_of(0, 0))
    q = torch.zeros((1, 2, 384, 128))
    with pytest.raises(SparseRouterError, match="equal Q/K shapes"):
        router.build_route(q, q[:, :1], layout_of(384, 128), 0.5)
    with pytest.raises(SparseRouterError, match="rank-4"):
        router.build_route(q[0], q[0], layout_of(384, 128), 0.5)
    with pytest.raises(ValueError, match="128-row query"):
        SparseTileRouter(q_tile=64, kv_tile=64)
    with pytest.raises(SparseSageError, match="requires CUDA"):
        B200SparseBackend()  # preflight: no device here
    backend = B200SparseBackend(check_device=False)
    with pytest.raises(SparseSageError, match="requires CUDA"):
        from h3_optimizations_b200 import runtime_options

        backend.prepare(q, q, q, layer_index=0, transformer_options=runtime_options(layout_of(384, 128)))
    with pytest.raises(TypeError):
        B200SparseBackend(config=object(), check_device=False)


def test_carrier_validation_mirrors_reference_messages():
    from h3_optimizations_b200.carriers import PreparedFusedQKV, validate_prepared_fused_qkv
    from h3_optimizations_b200.errors import FusedQKVError

    def make(**over):
        carrier = torch.zeros((1, 1, 64, 128), dtype=torch.int8)
        base = dict(
            q_int8=carrier.clone(), q_scale=torch.ones((1, 1, 1)), k_int8=carrier.clone(),
            k_scale=torch.ones((1, 1, 1)), v=torch.zeros((1, 1, 64, 128), dtype=torch.float16),
            q_summary=torch.zeros((1, 1, 1, 128), dtype=torch.float16),
            k_summary=torch.zeros((1, 1, 1, 128), dtype=torch.float16),
            output_dtype=torch.float16, sequence=64, heads=1, head_dim=128, layer_index=0,
        )
        base.update(over)
        return PreparedFusedQKV(**base)

    validate_prepared_fused_qkv(make())
    with pytest.raises(FusedQKVError, match="K scale shape"):
        validate_prepared_fused_qkv(make(k_scale=torch.ones((1, 1, 2))))
    with pytest.raises(FusedQKVError, match="must be INT8"):
        validate_prepared_fused_qkv(make(q_int8=torch.zeros((1, 1, 64, 128), dtype=torch.int16)))
    with pytest.raises(FusedQKVError, match="V is missing"):
        validate_prepared_fused_qkv(make(v=None))
    with pytest.raises(FusedQKVError, match="requires V scale"):
        validate_prepared_fused_qkv(make(v=None, v_carrier=torch.zeros((1, 1, 128, 128), dtype=torch.float8_e4m3fn)))
