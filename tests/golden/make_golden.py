"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference checkout exists (it is Python/torch and cannot travel
to the GPU box):

    python tests/golden/make_golden.py --reference /path/to/H3-Optimizations

Every fixture is the output of the reference's own function on seeded inputs
that the tests regenerate bit-for-bit (input checksums are stored beside the
outputs so that a platform whose RNG stream differs is detected rather than
misreported as a kernel bug):

* router_*.npz       SparseTileRouter.build_lut / build_compact_absolute_route
                     (attention/sparse/router.py, triton_route.py)
* quant_*.npz        sparse_sage._quantize_blocks (attention/sparse/sparse_sage.py:312-330)
* vstats.npz         fp8_v_stream.update_v_amax / finalize_v_scale
* schedule.json      config.resolve_video_budget tables
* float_ref.npz      benchmarks/bench_sparse_backends.sparse_float_reference
"""

from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))

from h3_optimizations_b200 import workloads  # noqa: E402


def checksum(*tensors):
    digest = hashlib.sha256()
    for t in tensors:
        digest.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return digest.hexdigest()


def layout_of(sequence, video_start):
    return SimpleNamespace(
        seq_len=sequence,
        video_range=(video_start, sequence),
        segments=((0, video_start, "text"), (video_start, sequence, "video")),
        video_shape=(1, 1, sequence - video_start),
        audio_t=0,
    )


def pack_mask(lut, valid):
    """Boolean (H,Tq,Tk) mask from a delta LUT, packed to bits."""
    absolute = torch.cumsum(lut[0], dim=-1)
    heads, q_tiles, kv_tiles = absolute.shape
    slots = torch.arange(kv_tiles)
    live = slots[None, None, :] < valid[0][..., None]
    hits = torch.zeros((heads, q_tiles, kv_tiles), dtype=torch.int32)
    hits.scatter_add_(2, absolute.clamp(0, kv_tiles - 1).long(), live.to(torch.int32))
    mask = hits > 0
    return np.packbits(mask.numpy(), axis=-1)


def router_case(ref, name, q, k, sequence, video_start, budget, out):
    router = ref.SparseTileRouter(q_tile=128, kv_tile=64)
    layout = layout_of(sequence, video_start)
    lut, valid, metadata = router.build_lut(q, k, layout, budget)
    payload = dict(
        mask_bits=pack_mask(lut, valid),
        valid=valid.numpy(),
        input_sha=np.array(checksum(q, k)),
        meta=np.array(json.dumps(metadata.as_dict())),
        sequence=sequence, video_start=video_start, budget=budget,
    )
    if lut.numel() <= 1_000_000:
        payload["lut"] = lut.numpy()
    np.savez_compressed(out / ("router_%s.npz" % name), **payload)
    print("router", name, metadata.as_dict())


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of the reference pack (the directory holding h3_optimizations/)")
    parser.add_argument("--skip-config1", action="store_true")
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    sys.path.insert(0, str(Path(args.reference) / "benchmarks"))
    from h3_optimizations.attention.sparse import fp8_v_stream, router as ref_router, triton_route
    from h3_optimizations.attention.sparse.config import HybridSparseConfig, resolve_video_budget
    from h3_optimizations.attention.sparse.sparse_sage import _quantize_blocks
    import bench_sparse_backends as ref_bench

    torch.set_num_threads(8)
    out = HERE

    # ---- router -----------------------------------------------------------
    spec = workloads.small_spec("r350", 2, 96, 254)
    q, k, _ = workloads.gaussian_qkv(spec, seed=11, widen=True)
    router_case(ref_router, "s350", q, k, 350, 96, 0.5, out)

    spec = workloads.small_spec("r1024", 3, 256, 768)
    q, k, _ = workloads.structured_qkv(spec, seed=5)
    router_case(ref_router, "s1024", q.float(), k.float(), 1024, 256, 0.3, out)

    q, k, _ = workloads.gaussian_qkv(workloads.CONFIG0, seed=0, widen=True)
    router_case(ref_router, "config0", q, k, 2304, 256, 0.3, out)

    # summaries entry + compact encoding (tests/test_triton_route.py geometry)
    torch.manual_seed(17)
    layout = layout_of(512, 192)
    router = ref_router.SparseTileRouter(q_tile=128, kv_tile=64)
    geo = router.geometry(layout)
    qs = torch.randn(1, 2, geo.q_tiles, 128, dtype=torch.float32)
    ks = torch.randn(1, 2, geo.kv_tiles, 128, dtype=torch.float32)
    lut, valid, _ = router.build_lut_from_summaries(qs, ks, layout, 0.3)
    route, _ = triton_route.build_compact_absolute_route(router, qs, ks, layout, 0.3)
    np.savez_compressed(out / "router_summaries512.npz", q_summary=qs.numpy(), k_summary=ks.numpy(),
                        lut=lut.numpy(), valid=valid.numpy(), route=route.numpy())

    if not args.skip_config1:
        q, k, _ = workloads.structured_qkv(workloads.CONFIG1, seed=0)
        router_case(ref_router, "config1", q.float(), k.float(), 33272, 512, 0.3, out)

    # ---- quantiser ----------------------------------------------------------
    spec = workloads.small_spec("q300", 2, 44, 256)
    for dtype, tag in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        q, k, _ = workloads.gaussian_qkv(spec, seed=3, dtype=torch.bfloat16, widen=dtype == torch.float32)
        q8, qs_ = _quantize_blocks(q, 128)
        k8, ks_ = _quantize_blocks(k, 64, subtract_mean=True)
        mean = k.mean(dim=-2, keepdim=True).float()
        np.savez_compressed(out / ("quant_%s.npz" % tag), q8=q8.numpy(), q_scale=qs_.numpy(), k8=k8.numpy(),
                            k_scale=ks_.numpy(), k_mean=mean.numpy(), input_sha=np.array(checksum(q, k)))

    # ---- V statistics -----------------------------------------------------------
    _, _, v = workloads.gaussian_qkv(spec, seed=3)
    amax = torch.zeros((1, 2, 128), dtype=torch.float32)
    fp8_v_stream.update_v_amax(amax, v[:, :, :128])
    fp8_v_stream.update_v_amax(amax, v[:, :, 128:])
    scale = fp8_v_stream.finalize_v_scale(amax.clone(), 448.0)
    np.savez_compressed(out / "vstats.npz", amax=amax.numpy(), scale=scale.numpy(), input_sha=np.array(checksum(v)))

    # ---- density schedule -----------------------------------------------------------
    tables = []
    cases = [
        dict(video_budget=0.5, denser_early_late_steps=True),
        dict(video_budget=0.85, denser_early_late_steps=True),
        dict(video_budget=0.3, early_steps=2, early_kv=0.5, late_steps=3, late_kv=0.7),
        dict(video_budget=0.3, early_steps=2, early_kv=0.5, late_steps=2, late_kv=0.5),
        dict(video_budget=0.7, early_steps=1, early_kv=0.2, late_steps=0, late_kv=0.4),
        dict(video_budget=0.3, early_steps=2, early_kv=0.4, late_steps=2, late_kv=0.6),
        dict(video_budget=0.2, layer_video_budgets=tuple(0.1 + i * 0.01 for i in range(50))),
        dict(video_budget=0.3),
    ]
    for kwargs in cases:
        config = HybridSparseConfig(**kwargs)
        for total in (3, 10, 20, 30):
            rows = []
            for step in range(-1, total + 1):
                layer = 7 if "layer_video_budgets" in kwargs else None
                rows.append([step, resolve_video_budget(config, step, total, layer)])
            tables.append(dict(config={k: (list(v) if isinstance(v, tuple) else v) for k, v in kwargs.items()},
                               total_steps=total, budgets=rows))
    (out / "schedule.json").write_text(json.dumps(tables))

    # ---- float sparse reference ------------------------------------------------------
    spec = workloads.small_spec("f384", 1, 128, 256)
    q, k, v = workloads.gaussian_qkv(spec, seed=9, widen=True)
    layout = layout_of(384, 128)
    lut, valid, _ = router.build_lut(q, k, layout, 0.5)
    ref = ref_bench.sparse_float_reference(torch, q, k, v, lut, valid, 128, 64)
    np.savez_compressed(out / "float_ref.npz", out=ref.numpy(), lut=lut.numpy(), valid=valid.numpy(),
                        input_sha=np.array(checksum(q, k, v)))
    print("done")


if __name__ == "__main__":
    main()
