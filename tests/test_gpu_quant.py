"""Carrier quantisation kernels against the oracle and the reference fixtures
(bit-exact for INT8 codes, scales and FP8 bytes).  Needs a B200."""

import numpy as np
import pytest
import torch

from h3_optimizations_b200 import workloads
from oracle import h3_oracle as oracle
from tests.helpers import checksum

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(native_lib):
    from h3_optimizations_b200 import ops as module

    return module


def _q300(tag):
    spec = workloads.small_spec("q300", 2, 44, 256)
    return workloads.gaussian_qkv(spec, seed=3, dtype=torch.bfloat16, widen=tag == "f32")


@pytest.mark.parametrize("tag", ["bf16", "f32"])
def test_qk_codes_and_scales_match_reference_fixture(ops, golden_dir, tag):
    data = np.load(golden_dir / ("quant_%s.npz" % tag))
    q, k, _ = _q300(tag)
    if checksum(q, k) != str(data["input_sha"]):
        q8_ref, qs_ref = oracle.quantize_blocks(q, 128)
        k8_ref, ks_ref = oracle.quantize_blocks(k, 64, subtract_mean=True)
        mean = k.mean(dim=-2, keepdim=True).float().reshape(1, 2, 128)
    else:
        q8_ref, qs_ref = torch.from_numpy(data["q8"]), torch.from_numpy(data["q_scale"])
        k8_ref, ks_ref = torch.from_numpy(data["k8"]), torch.from_numpy(data["k_scale"])
        mean = torch.from_numpy(data["k_mean"]).reshape(1, 2, 128)
    q8, qs, _ = ops.quant_qk_blocks(q.cuda(), 128)
    k8, ks, _ = ops.quant_qk_blocks(k.cuda(), 64, mean=mean.cuda().contiguous())
    assert torch.equal(q8.cpu(), q8_ref) and torch.equal(qs.cpu(), qs_ref)
    assert torch.equal(k8.cpu(), k8_ref) and torch.equal(ks.cpu(), ks_ref)


def test_qk_known_answers_of_reference_tests(ops):
    # reference tests/test_triton_sparse_qkv.py:51-63
    q = torch.zeros(1, 1, 128, 128, dtype=torch.float16)
    k = torch.zeros_like(q)
    q[..., 0, 0] = 127.0
    k[..., 0, 1] = 63.5
    q8, qs, _ = ops.quant_qk_blocks(q.cuda(), 128)
    k8, ks, _ = ops.quant_qk_blocks(k.cuda(), 64)
    assert abs(float(qs[0, 0, 0]) - 1.0) < 1e-4 and abs(float(ks[0, 0, 0]) - 0.5) < 1e-4
    assert int(q8[0, 0, 0, 0]) == 127 and int(k8[0, 0, 0, 1]) == 127
    # an all-zero block quantises to zeros with the epsilon scale
    assert float(ks[0, 0, 1]) == pytest.approx(1e-7) and int(k8[0, 0, 64:].abs().max()) == 0


@pytest.mark.parametrize("sequence", [1, 63, 64, 129, 300, 1000])
def test_ragged_tails_and_strided_views(ops, sequence):
    gen = torch.Generator().manual_seed(sequence)
    heads = 3
    token_major = torch.randn((sequence, heads * 128), generator=gen).to(torch.bfloat16)
    x = token_major.view(sequence, heads, 128).permute(1, 0, 2).unsqueeze(0)  # HND view, stride_s = H*128
    for block in (128, 64):
        ref8, ref_scale = oracle.quantize_blocks(x, block)
        got8, got_scale, summary = ops.quant_qk_blocks(x.cuda(), block, summary_dtype=torch.float64)
        assert torch.equal(got8.cpu(), ref8) and torch.equal(got_scale.cpu(), ref_scale)
        # each thread adds its (at most 8) rows in fp32 before the FP64 reduction, so the
        # mean is exact to fp32 rounding of those partial sums, not to the last FP64 bit
        exact = oracle.mean_pool(x.double(), block)
        assert torch.allclose(summary.cpu(), exact, rtol=0, atol=2e-7)
        bf = ops.tile_means(x.cuda(), block, dtype=torch.bfloat16)
        assert torch.allclose(bf.cpu().float(), oracle.block_summaries(x, block).float(), rtol=0, atol=1e-2)


def test_chunked_packing_equals_one_shot(ops):
    # reference tests/test_chunked_sparse_qkv.py:93-133 - rows as values, 128-row chunks
    rows = torch.arange(0, 300, dtype=torch.float32).view(1, 1, -1, 1).expand(1, 2, -1, 128).contiguous()
    for block, offset, expect in ((128, 0.0, 277.5), (64, 100.0, 377.5)):
        x = (rows + offset).cuda()
        out = torch.empty((1, 2, 300, 128), dtype=torch.int8, device="cuda")
        blocks = (300 + block - 1) // block
        scale = torch.empty((1, 2, blocks), dtype=torch.float32, device="cuda")
        summary = torch.empty((1, 2, blocks, 128), dtype=torch.float32, device="cuda")
        for start in range(0, 300, 128):
            end = min(start + 128, 300)
            ops.quant_qk_blocks_into(x[:, :, start:end], out, scale, summary, block=block, row_start=start)
        whole8, whole_scale, whole_summary = ops.quant_qk_blocks(x, block, summary_dtype=torch.float32)
        assert torch.equal(out, whole8) and torch.equal(scale, whole_scale) and torch.equal(summary, whole_summary)
        assert float(summary[0, 0, -1, 0]) == expect
        ref8, ref_scale = oracle.quantize_blocks(x.cpu(), block)
        assert torch.equal(out.cpu(), ref8) and torch.equal(scale.cpu(), ref_scale)


def test_column_stats_and_v_carrier(ops, golden_dir):
    data = np.load(golden_dir / "vstats.npz")
    q, k, v = workloads.gaussian_qkv(workloads.small_spec("q300", 2, 44, 256), seed=3)
    k_mean, v_scale = ops.column_stats(k.cuda(), v.cuda())
    if checksum(v) == str(data["input_sha"]):
        assert np.array_equal(v_scale.cpu().numpy(), data["scale"])
    ref_carrier, ref_scale = oracle.v_fp8_carrier(v)
    assert torch.equal(v_scale.cpu(), ref_scale)
    # the mean agrees with torch's to one bf16 ulp (the summation orders differ)
    ref_mean = k.mean(dim=-2).float()
    assert float((k_mean.cpu() - ref_mean).abs().max()) <= 2.0 ** -8 * float(ref_mean.abs().max()) + 1e-6
    carrier, scale = ops.quant_v_fp8(v.cuda(), v_scale)
    assert tuple(carrier.shape) == (1, 2, 128, 384)
    assert torch.equal(carrier.cpu().view(torch.uint8), ref_carrier.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_v_carrier_chunked_and_dtypes(ops, dtype):
    gen = torch.Generator().manual_seed(5)
    sequence, heads = 700, 2
    v = (torch.randn((1, heads, sequence, 128), generator=gen) * 3).to(dtype)
    ref_carrier, ref_scale = oracle.v_fp8_carrier(v)
    vc = v.cuda()
    _, v_scale = ops.column_stats(None, vc)
    assert torch.equal(v_scale.cpu(), ref_scale)
    carrier = ops.allocate_v_carrier(sequence, heads, "cuda")
    carrier.view(torch.uint8).fill_(0x55)  # the kernel must overwrite the padding itself
    for start in range(0, sequence, 256):
        end = min(start + 256, sequence)
        ops.quant_v_fp8_into(vc[:, :, start:end], v_scale, carrier, row_start=start, sequence_total=sequence)
    assert torch.equal(carrier.cpu().view(torch.uint8), ref_carrier.view(torch.uint8))


def test_invalid_arguments_are_rejected_on_the_host(ops):
    from h3_optimizations_b200._native import NativeError

    x = torch.zeros((1, 1, 128, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NativeError, match="block must be 128 or 64"):
        ops.quant_qk_blocks(x, 32)
    out = torch.empty((1, 1, 256, 128), dtype=torch.int8, device="cuda")
    scale = torch.empty((1, 1, 2), dtype=torch.float32, device="cuda")
    with pytest.raises(NativeError, match="not a multiple of the block"):
        ops.quant_qk_blocks_into(x, out, scale, None, block=128, row_start=64)
    with pytest.raises(NativeError, match="partial tile"):
        ops.quant_qk_blocks_into(x[:, :, :100], out, scale, None, block=128, row_start=0)
    with pytest.raises(NativeError, match="CUDA tensor"):
        ops.quant_qk_blocks(x.cpu(), 128)
    misaligned = torch.zeros((1, 1, 128, 136), dtype=torch.bfloat16, device="cuda")[..., 4:132]
    with pytest.raises(NativeError, match="aligned"):
        ops.quant_qk_blocks(misaligned, 128)
