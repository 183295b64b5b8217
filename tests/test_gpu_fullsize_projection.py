"""The chunked QKV projection at its full benchmark shape.  Needs a B200.

33272 tokens x 3072 channels -> 24 heads x (Q, K, V) x 128, nine chunks of 4096
rows of which the last holds 504 (three full 128-row tiles and one of 120
rows).  The CPU oracle cannot redo all 1.9 TOP in a test, so it checks

* the de-quantised bf16 projection bit for bit on a sample of rows of every
  chunk (first, last, tile edges) over all 9216 output columns, and
* every carrier of two heads (first and last) over the whole sequence: INT8 Q/K
  codes and scales, tile means, FP8 V bytes and scale."""

from types import SimpleNamespace

import pytest
import torch

from h3_optimizations_b200 import workloads
from oracle import h3_oracle as oracle

pytestmark = pytest.mark.gpu

SEQUENCE, HIDDEN, HEADS, CHUNK = 33272, 3072, 24, 4096


@pytest.fixture(scope="module")
def operands(native_lib):
    x, w, w_scale = workloads.projection_inputs(SEQUENCE, hidden=HIDDEN, heads=HEADS, seed=0)
    x_i8, x_scale = oracle.convrot_quantize_rows(x)
    return x, w, w_scale, x_i8, x_scale


def test_rotation_and_gemm_on_sampled_rows_of_every_chunk(operands):
    from h3_optimizations_b200 import ops

    x, w, w_scale, x_i8, x_scale = operands
    xd, wd, wsd = x.cuda(), w.cuda(), w_scale.cuda()
    codes, scale = ops.convrot_quant_rows(xd)
    assert torch.equal(codes.cpu(), x_i8) and torch.equal(scale.cpu(), x_scale), "ConvRot codes of all 33272 rows"
    staging = torch.empty((3 * HEADS, SEQUENCE, 128), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rows = []
    for start in range(0, SEQUENCE, CHUNK):
        end = min(start + CHUNK, SEQUENCE)
        ops.qkv_gemm_chunk(codes[start:end], scale[start:end], wd, wsd, staging, row_start=start, status=status)
        rows += [start, start + 127, start + 128, (start + end) // 2, end - 1]
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    rows = sorted(set(rows))
    index = torch.tensor(rows)
    reference = oracle.qkv_project_int8(x_i8[index], x_scale[index], w, w_scale)          # (len(rows), 9216) bf16
    got = staging[:, index.cuda()].permute(1, 0, 2).reshape(len(rows), 3 * HEADS * 128).cpu()
    assert torch.equal(got.view(torch.int16), reference.view(torch.int16))


@pytest.mark.parametrize("smooth_k", [True, False], ids=["smoothed K", "plain K"])
def test_carriers_of_two_heads_over_the_whole_sequence(operands, smooth_k):
    from h3_optimizations_b200 import ChunkedSparseQKVProjector, ops

    x, w, w_scale, x_i8, x_scale = operands
    module = SimpleNamespace(heads=HEADS, head_dim=128, qkv_weight_int8=w.cuda(), qkv_weight_scale=w_scale.cuda())
    prepared = ChunkedSparseQKVProjector(chunk_rows=CHUNK, smooth_k=smooth_k).project(
        module, x.cuda(), None, layer_index=0, transformer_options={})
    torch.cuda.synchronize()
    for head in (0, HEADS - 1):
        columns = torch.cat([torch.arange(128) + (kind * HEADS + head) * 128 for kind in range(3)])
        y = oracle.qkv_project_int8(x_i8, x_scale, w[columns], w_scale[columns])           # (S, 384) bf16
        q, k, v = oracle.split_heads_hnd(y, 1)
        q8, qs = oracle.quantize_blocks(q, 128)
        assert torch.equal(prepared.q_int8[:, head:head + 1].cpu(), q8), "Q codes, head %d" % head
        assert torch.equal(prepared.q_scale[:, head:head + 1].cpu(), qs)
        if smooth_k:
            # the device mean is a sum in FP64 rounded once; torch's bf16 mean can differ in the
            # last place of a channel, which moves codes of that channel by one step
            device_mean, _ = ops.column_stats(k.cuda().contiguous(), None)
            k8, ks = oracle.quantize_blocks(k, 64, mean=device_mean.cpu())
            own8, _ = oracle.quantize_blocks(k, 64, subtract_mean=True)
            differing = int((own8 != k8).sum())
            print("head %d: %d of %d K codes differ when the oracle takes its own bf16 mean (%.2e)"
                  % (head, differing, k8.numel(), differing / k8.numel()))
            assert differing <= 0.02 * k8.numel()
            assert int((own8.int() - k8.int()).abs().max()) <= 1
        else:
            k8, ks = oracle.quantize_blocks(k, 64)
        assert torch.equal(prepared.k_int8[:, head:head + 1].cpu(), k8), "K codes, head %d" % head
        assert torch.equal(prepared.k_scale[:, head:head + 1].cpu(), ks)
        vc, vs = oracle.v_fp8_carrier(v)
        assert torch.equal(prepared.v_scale[:, head:head + 1].cpu(), vs)
        assert torch.equal(prepared.v_carrier[:, head:head + 1].cpu().view(torch.uint8), vc.view(torch.uint8))
        assert torch.allclose(prepared.q_summary[:, head:head + 1].cpu(), oracle.block_summaries(q, 128, torch.float32),
                              atol=1e-5)
        assert torch.allclose(prepared.k_summary[:, head:head + 1].cpu(), oracle.block_summaries(k, 64, torch.float32),
                              atol=1e-5)
