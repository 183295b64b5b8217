"""Dense tensor-core GEMM, FP8 row quantiser, out_proj behind the attention and
the chunked FP8 MLP.  Needs a B200.

These are floating-point kernels: the check is a torch FP32 (FP64 where cheap)
evaluation of the same operands.  Tolerances: the accumulation is FP32 in both,
so what differs is the order of the additions and the final rounding to bf16
(relative 2^-8); the bound used is 1.5 bf16 ulps of the largest magnitude in
the row plus the same relative to the element."""

from types import SimpleNamespace

import pytest
import torch

from h3_optimizations_b200 import workloads
from oracle import h3_oracle as oracle

pytestmark = pytest.mark.gpu

BF16_ULP = 2.0 ** -8


def _close(got, want, scale=1.5):
    got, want = got.float().cpu(), want.float().cpu()
    bound = scale * BF16_ULP * (want.abs() + want.abs().amax(dim=-1, keepdim=True) * 0.02) + 1e-6
    worst = ((got - want).abs() / bound).max()
    assert float(worst) <= 1.0, "largest error is %.2f times the bound" % float(worst)


@pytest.fixture(scope="module")
def ops(native_lib):
    from h3_optimizations_b200 import ops as module

    return module


@pytest.mark.parametrize("rows,n_out,k", [(128, 256, 128), (300, 3072, 3072), (4096, 1000, 1024), (77, 136, 384)])
def test_bf16_gemm_with_bias(ops, rows, n_out, k):
    gen = torch.Generator().manual_seed(rows)
    a = torch.randn((rows, k), generator=gen).to(torch.bfloat16)
    b = (torch.randn((n_out, k), generator=gen) * k ** -0.5).to(torch.bfloat16)
    bias = torch.randn((n_out,), generator=gen)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = ops.dense_gemm(a.cuda(), b.cuda(), bias=bias.cuda(), status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    want = a.double() @ b.double().T + bias.double()
    _close(out, want)
    # a strided output (columns of a wider matrix) and no bias
    wide = torch.full((rows, n_out + 64), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.dense_gemm(a.cuda(), b.cuda(), out=wide[:, :n_out])
    torch.cuda.synchronize()
    _close(wide[:, :n_out], a.double() @ b.double().T)
    assert bool(torch.isnan(wide[:, n_out:].float()).all()), "columns beyond n_out stay untouched"


def test_int8_and_fp8_operands_with_scales_and_gelu(ops):
    gen = torch.Generator().manual_seed(5)
    rows, n_out, k = 520, 768, 1024
    a8 = torch.randint(-127, 128, (rows, k), generator=gen, dtype=torch.int16).to(torch.int8)
    b8 = torch.randint(-127, 128, (n_out, k), generator=gen, dtype=torch.int16).to(torch.int8)
    rs = torch.rand((rows,), generator=gen) * 1e-2 + 1e-3
    cs = torch.rand((n_out,), generator=gen) * 1e-2 + 1e-3
    out = ops.dense_gemm(a8.cuda(), b8.cuda(), row_scale=rs.cuda(), col_scale=cs.cuda())
    want = (a8.double() @ b8.double().T) * rs.double()[:, None] * cs.double()[None, :]
    _close(out, want)

    af = (torch.randn((rows, k), generator=gen) * 3).to(torch.float8_e4m3fn)
    bf = (torch.randn((n_out, k), generator=gen) * 3).to(torch.float8_e4m3fn)
    bias = torch.randn((n_out,), generator=gen)
    out = ops.dense_gemm(af.cuda(), bf.cuda(), row_scale=rs.cuda(), col_scale=cs.cuda(), bias=bias.cuda(),
                         activation="gelu_tanh")
    pre = (af.double() @ bf.double().T) * rs.double()[:, None] * cs.double()[None, :] + bias.double()
    want = torch.nn.functional.gelu(pre, approximate="tanh")
    _close(out, want)


def test_fp8_row_quantiser(ops):
    gen = torch.Generator().manual_seed(9)
    x = (torch.randn((300, 12288), generator=gen) * torch.rand((300, 1), generator=gen) * 4).to(torch.bfloat16)
    x[7] = 0
    codes, scale = ops.quant_rows_fp8(x.cuda())
    want_scale = (x.float().abs().amax(dim=1) / 448.0).clamp_min(1e-20)
    assert torch.equal(scale.cpu(), want_scale)
    want = (x.float() / want_scale[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert torch.equal(codes.cpu().view(torch.uint8), want.view(torch.uint8))


def test_out_proj_behind_the_attention(ops):
    """`execute_projected`: attention + out_proj as one backend call returning (S, hidden)."""
    from h3_optimizations_b200 import B200SparseBackend, HybridSparseConfig, runtime_options
    from h3_optimizations_b200.attention_forward import make_forward

    spec = workloads.small_spec("proj", 2, 192, 832)
    q, k, v = (t.cuda() for t in workloads.gaussian_qkv(spec, seed=3))
    gen = torch.Generator().manual_seed(4)
    linear = torch.nn.Linear(256, 384, bias=True).to(torch.bfloat16)
    with torch.no_grad():
        linear.weight.copy_((torch.randn((384, 256), generator=gen) * 256 ** -0.5).to(torch.bfloat16))
    linear = linear.cuda()
    module = SimpleNamespace(out_proj=linear, heads=2, head_dim=128)
    backend = B200SparseBackend(HybridSparseConfig(video_budget=0.3))
    options = runtime_options(spec.layout())
    prepared = backend.prepare(q, k, v, layer_index=0, transformer_options=options)
    rows = backend.execute_projected(module, prepared)
    attention = backend.execute(prepared)
    torch.cuda.synchronize()
    assert rows is not None and tuple(rows.shape) == (1024, 384) and rows.dtype == torch.bfloat16
    flat = attention.permute(0, 2, 1, 3).reshape(1024, 256)
    want = flat.double() @ linear.weight.detach().double().T + linear.bias.detach().double()
    _close(rows, want)
    # a projection this entry does not take (fp32 weight): the caller falls back to execute + module.out_proj
    assert backend.execute_projected(SimpleNamespace(out_proj=torch.nn.Linear(256, 384).cuda(), heads=2, head_dim=128),
                                     prepared) is None


def test_chunked_fp8_mlp(ops):
    from h3_optimizations_b200.mlp import ChunkedFP8MLP, quantize_weight_rows_fp8

    gen = torch.Generator().manual_seed(11)
    tokens, hidden, ffn = 700, 512, 2048
    x = torch.randn((tokens, hidden), generator=gen).to(torch.bfloat16)
    w1 = torch.randn((ffn, hidden), generator=gen) * 0.02
    w2 = torch.randn((hidden, ffn), generator=gen) * 0.02
    b1 = torch.randn((ffn,), generator=gen) * 0.1
    b2 = torch.randn((hidden,), generator=gen) * 0.1
    mlp = ChunkedFP8MLP(w1, b1, w2, b2, chunk_rows=256).to("cuda")
    out = mlp(x.cuda())
    torch.cuda.synchronize()

    # the same arithmetic on the host: per-row E4M3 operands, products and sums in FP64, bf16 intermediate
    def rows_fp8(t):
        scale = (t.float().abs().amax(dim=1) / 448.0).clamp_min(1e-20)
        return (t.float() / scale[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn), scale

    w1q, w1s = quantize_weight_rows_fp8(w1)
    w2q, w2s = quantize_weight_rows_fp8(w2)
    xq, xs = rows_fp8(x)
    h = torch.nn.functional.gelu((xq.double() @ w1q.double().T) * xs.double()[:, None] * w1s.double()[None, :] + b1.double(),
                                 approximate="tanh").to(torch.bfloat16)
    hq, hs = rows_fp8(h)
    want = (hq.double() @ w2q.double().T) * hs.double()[:, None] * w2s.double()[None, :] + b2.double()
    # the bf16 rounding of h can fall the other way in a few places, which moves an E4M3 code of h by
    # one step (2^-4 of that element); the output is a sum over 2048 of them
    _close(out, want, scale=3.0)
    full = torch.nn.functional.gelu(x.double() @ w1.double().T + b1.double(), approximate="tanh") @ w2.double().T + b2.double()
    m = oracle.compare(out.float().cpu(), full.float())
    print("FP8 MLP vs FP64 MLP on unquantised operands:", m)
    assert m["cosine"] >= 0.998  # reported: what E4M3 operands cost against an unquantised FP64 MLP
