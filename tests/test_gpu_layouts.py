"""Mixed-modality layout, batch > 1 and the 76112-token sequence.  Needs a B200.

* text + reference conditioning + audio + video (the packed order the reference
  uses, runtime/layout.py:116-118: video last, audio before it): every tile that
  is not entirely video - 24 query tiles, 48 KV tiles - stays dense, the mask is
  compared bit for bit with the reference's own router run on the host from
  oracle/_ref, and a batch of two goes through ``backend.forward``;
* the 76112-token sequence at 30 %: a sample of (head, query tile) pairs against
  the CPU oracle."""

import dataclasses

import pytest
import torch

from h3_optimizations_b200 import workloads
from oracle import h3_oracle as oracle
from oracle import ref_bridge

pytestmark = pytest.mark.gpu

GATE_COS, GATE_REL = 0.999, 2e-2


def _carriers(q, k, v):
    q8, qs = oracle.quantize_blocks(q, 128)
    k8, ks = oracle.quantize_blocks(k, 64, subtract_mean=True)
    vc, vs = oracle.v_fp8_carrier(v)
    return q8, qs, k8, ks, vc, vs


def test_mixed_modality_layout_and_batch_of_two(native_lib):
    from h3_optimizations_b200 import B200SparseBackend, HybridSparseConfig, runtime_options

    heads = 2
    spec = dataclasses.replace(workloads.CONFIG4, heads=heads)
    assert spec.sequence == 35832 and spec.video_range == (3072, 35832)
    batch = [workloads.structured_qkv(spec, seed=seed) for seed in (0, 1)]
    q, k, v = (torch.cat([b[i] for b in batch], dim=0) for i in range(3))      # (2, H, S, 128)
    backend = B200SparseBackend(HybridSparseConfig(video_budget=0.3))
    options = runtime_options(spec.layout())
    with pytest.raises(Exception, match="batch 1"):
        backend.prepare(q.cuda(), k.cuda(), v.cuda(), layer_index=0, transformer_options=options)
    out = backend.forward(q.cuda(), k.cuda(), v.cuda(), layer_index=0, transformer_options=options)
    torch.cuda.synchronize()
    backend.check_status()
    assert tuple(out.shape) == (2, heads, spec.sequence, 128)

    geo = oracle.geometry(spec.sequence, 3072)
    assert (geo.pure_video_q_start, geo.pure_video_kv_start, geo.q_tiles, geo.kv_tiles) == (24, 48, 280, 560)
    tiles = [0, 5, 23, 24, 25, 150, 279]   # text, reference, audio (dense), first video tiles, middle, ragged last
    rows = torch.cat([torch.arange(t * 128, min(t * 128 + 128, spec.sequence)) for t in tiles])
    for b in range(2):
        qb, kb, vb = (t[b:b + 1] for t in (q, k, v))
        prepared = backend.prepare(qb.cuda(), kb.cuda(), vb.cuda(), layer_index=0, transformer_options=options)
        route = prepared.sparse.route.indices.cpu()
        assert route.shape[-1] == 48 + 154
        leading = torch.arange(48, dtype=torch.int32).expand(1, heads, 256, 48)
        assert torch.equal(route[..., :48], leading), "the 48 context tiles lead every routed row"
        if ref_bridge.available():
            lut, valid, meta = ref_bridge.build_lut(qb.float(), kb.float(), spec.sequence, 3072, 0.3,
                                                    segments=spec.segments)
            absolute = ref_bridge.bench_module().absolute_lut(torch, lut)
            assert torch.equal(absolute[0, :, 24:, :202], route[0]), "mask differs from the reference router's"
            assert bool((valid[0, :, :24] == 560).all()) and bool((valid[0, :, 24:] == 202).all())
            assert meta.dense_q_tiles == 24 and meta.retained_video_kv_tiles == 154
        gate = oracle.sparse_attention_int8_fp8(*_carriers(qb[:, :1], kb[:, :1], vb[:, :1]), geo, route[:, :1],
                                                q_tile_subset=tiles)
        m = oracle.compare(out[b:b + 1, :1].float().cpu()[:, :, rows], gate[:, :, rows])
        assert m["cosine"] >= GATE_COS and m["rel_max_abs"] <= GATE_REL, (b, m)


def test_long_sequence_sampled_against_the_oracle(native_lib):
    from h3_optimizations_b200 import B200SparseBackend, HybridSparseConfig, runtime_options

    heads = 2
    spec = dataclasses.replace(workloads.CONFIG3, heads=heads)
    q, k, v = workloads.structured_qkv(spec, seed=0)
    backend = B200SparseBackend(HybridSparseConfig(video_budget=0.3))
    prepared = backend.prepare(q.cuda(), k.cuda(), v.cuda(), layer_index=0,
                               transformer_options=runtime_options(spec.layout()))
    out = backend.execute(prepared)
    torch.cuda.synchronize()
    backend.check_status()
    sparse = prepared.sparse
    assert sparse.route.route_len == 8 + 355 and sparse.metadata["retained_video_kv_tiles"] == 355
    geo = oracle.geometry(spec.sequence, 512)
    _, _, _, oracle_route = oracle.build_route(q[:, 1:].float(), k[:, 1:].float(), spec.sequence, 512, 0.3)
    route = sparse.route.indices.cpu()
    assert torch.equal(route[:, 1:], oracle_route), "router mask of head 1 (591 rows of 1182 scores)"
    tiles = [0, 3, 4, 300, 593, 594]   # dense text tiles, first routed, middle, last full, ragged last
    rows = torch.cat([torch.arange(t * 128, min(t * 128 + 128, spec.sequence)) for t in tiles])
    gate = oracle.sparse_attention_int8_fp8(*_carriers(q[:, 1:], k[:, 1:], v[:, 1:]), geo, route[:, 1:], q_tile_subset=tiles)
    m = oracle.compare(out[:, 1:].float().cpu()[:, :, rows], gate[:, :, rows])
    assert m["cosine"] >= GATE_COS and m["rel_max_abs"] <= GATE_REL, m
