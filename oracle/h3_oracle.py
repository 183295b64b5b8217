"""CPU oracle for the H3 sparse-attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, with torch CPU ops, the arithmetic of the reference pack
(Pizzawookiee/H3-Optimizations) for the path

    QKV projection -> INT8/FP8 carriers -> block router -> block-sparse attention.

It is the checker the CUDA path is compared against.  Only the test-suite, the
smoke entry and the `cpu_baseline` / `--impl reference` legs of the benchmark
may import it; the product package never does.

Parity status of each function (what pins it):

* router (`geometry`, `retained_tiles`, `mean_pool`, `select_tiles`,
  `compact_route`, `delta_lut`), `quantize_blocks`, `resolve_video_budget`:
  PINNED - checked against the reference's own functions run in a container
  that has the reference checked out (fixtures in tests/golden, produced by
  tests/golden/make_golden.py) and against the known answers of the reference
  unit tests (tests/test_router.py, tests/test_triton_route.py,
  tests/test_triton_sparse_qkv.py, tests/test_chunked_sparse_qkv.py,
  tests/test_sparse_density.py).
* `v_fp8_carrier`: scale/clamp helpers are pinned against
  attention/sparse/fp8_v_stream.py (`update_v_amax`, `finalize_v_scale`); the
  quantising kernel of the reference is Triton-only, so the element cast is a
  restatement of fp8_v_stream.py:50-55.
* `sparse_attention_int8_fp8`: PARITY UNPINNED.  The reference's Sparse Sage
  kernel lives in the third-party package spas_sage_attn (thu-ml/SpargeAttn
  @ ae5b629ebb41e41f86b3ea2ab5a3283f13ac151a), which is not vendored; no
  reference test pins any attention output.  The restatement follows the
  in-repo INT8 Triton kernel (attention/sparse/triton_sparse_kernels.py:121-203)
  with the V operand taken from the FP8 carrier.
* `convrot_quantize_rows`, `qkv_project_int8`: PARITY UNPINNED for the rotation
  (it lives in comfy_kitchen); the GEMM + dequantisation follow
  attention/sparse/fused_qkv.py:198-223 and are pinned only by construction
  (integer GEMM is exact).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

Q_TILE = 128
KV_TILE = 64
HEAD_DIM = 128
LOG2E = 1.4426950408889634
FP8_E4M3_MAX = 448.0
# FP8 probabilities are taken relative to 2^(ceil(rowmax) - 7): the largest is
# in (64, 128], which leaves E4M3 (max 448, min normal 2^-6) thirteen octaves below.
P_EXPONENT_OFFSET = 7.0


# --------------------------------------------------------------------------
# Density schedule (reference: attention/sparse/config.py:94-129)
# --------------------------------------------------------------------------

def resolve_video_budget(
    video_budget,
    step_index,
    total_steps,
    *,
    layer_index=None,
    early_steps=None,
    early_kv=None,
    late_steps=None,
    late_kv=None,
    denser_early_late_steps=False,
    layer_video_budgets=None,
):
    """Budget for one (sampler step, layer).  config.py:94-129."""
    if layer_video_budgets is not None:
        if layer_index is None:
            raise ValueError("layer_index is required for static per-layer budgets")
        return float(layer_video_budgets[int(layer_index)])
    budget = float(video_budget)
    step_index = int(step_index)
    total_steps = int(total_steps)
    if step_index < 0 or total_steps <= 0 or step_index >= total_steps:
        return budget
    if early_steps is not None:
        in_early = step_index < int(early_steps)
        in_late = step_index >= total_steps - int(late_steps)
        if in_early and in_late:
            return max(float(early_kv), float(late_kv))
        if in_early:
            return float(early_kv)
        if in_late:
            return float(late_kv)
        return budget
    if not denser_early_late_steps:
        return budget
    if step_index < 2 or step_index >= total_steps - 2:
        return min(1.0, budget + 0.30)
    return budget


# --------------------------------------------------------------------------
# Router (reference: attention/sparse/router.py)
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class Geometry:
    """Tile geometry.  router.py:59-74,124-160, generalised to a video range
    that need not end the sequence: a tile is *pure video* when every row it
    covers lies inside ``[video_start, video_stop)``; with ``video_stop ==
    sequence`` this is exactly the reference rule (the ragged tail tile counts
    as pure video there)."""

    sequence: int
    q_tiles: int
    kv_tiles: int
    pure_video_q_start: int
    pure_video_q_stop: int
    pure_video_kv_start: int
    pure_video_kv_stop: int

    @property
    def pure_video_q_tiles(self):
        return self.pure_video_q_stop - self.pure_video_q_start

    @property
    def pure_video_kv_tiles(self):
        return self.pure_video_kv_stop - self.pure_video_kv_start

    @property
    def context_kv_tiles(self):
        return self.kv_tiles - self.pure_video_kv_tiles


def _ceil_div(a, b):
    return (a + b - 1) // b


def geometry(sequence, video_start, video_stop=None, q_tile=Q_TILE, kv_tile=KV_TILE):
    sequence = int(sequence)
    video_start = int(video_start)
    video_stop = sequence if video_stop is None else int(video_stop)
    if sequence <= 0:
        raise ValueError("packed sequence is empty")
    if not (0 <= video_start < video_stop <= sequence):
        raise ValueError("invalid video range")
    q_tiles = _ceil_div(sequence, q_tile)
    kv_tiles = _ceil_div(sequence, kv_tile)

    def stop_tile(tile, tiles):
        return tiles if video_stop == sequence else video_stop // tile

    geo = Geometry(
        sequence=sequence,
        q_tiles=q_tiles,
        kv_tiles=kv_tiles,
        pure_video_q_start=_ceil_div(video_start, q_tile),
        pure_video_q_stop=stop_tile(q_tile, q_tiles),
        pure_video_kv_start=_ceil_div(video_start, kv_tile),
        pure_video_kv_stop=stop_tile(kv_tile, kv_tiles),
    )
    if geo.pure_video_q_tiles <= 0:
        raise ValueError("packed layout has no pure-video query tiles")
    if geo.pure_video_kv_tiles <= 0:
        raise ValueError("packed layout has no pure-video KV tiles")
    return geo


def retained_tiles(video_budget, geo):
    """router.py:180-193 - host double arithmetic, math.ceil."""
    pure = geo.pure_video_kv_tiles
    return min(pure, max(1, int(math.ceil(float(video_budget) * pure))))


def mask_metadata(geo, video_budget, retained):
    """router.py:195-217."""
    pure_q = geo.pure_video_q_tiles
    pure_kv = geo.pure_video_kv_tiles
    sparse_q = pure_q if retained < pure_kv else 0
    non_video_kv = geo.kv_tiles - pure_kv
    true_blocks = (geo.q_tiles - pure_q) * geo.kv_tiles + pure_q * (non_video_kv + retained)
    return dict(
        requested_video_budget=float(video_budget),
        actual_video_tile_density=float(retained) / pure_kv,
        full_mask_density=float(true_blocks) / (geo.q_tiles * geo.kv_tiles),
        dense_q_tiles=geo.q_tiles - sparse_q,
        sparse_q_tiles=sparse_q,
        q_tiles=geo.q_tiles,
        kv_tiles=geo.kv_tiles,
        pure_video_q_tiles=pure_q,
        pure_video_kv_tiles=pure_kv,
        retained_video_kv_tiles=retained,
        density_mode="fixed",
    )


def mean_pool(x, block):
    """Mean over each block's real rows, in x.dtype.  router.py:162-178."""
    sequence = x.shape[-2]
    full = sequence // block
    remainder = sequence % block
    pieces = []
    if full:
        pieces.append(
            x[..., : full * block, :]
            .reshape(*x.shape[:-2], full, block, x.shape[-1])
            .mean(dim=-2)
        )
    if remainder:
        pieces.append(x[..., full * block:, :].mean(dim=-2, keepdim=True))
    return pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=-2)


def select_tiles(q_summary, k_summary, geo, retained, *, q_chunk_tiles=64):
    """Top-``retained`` pure-video KV tiles per pure-video query tile, as
    ascending absolute tile indices ``(B,H,pure_q,retained)`` int32.
    router.py:38-56 (chunked matmul + topk), 453-457 (offset, sort)."""
    q = q_summary[..., geo.pure_video_q_start:geo.pure_video_q_stop, :]
    k = k_summary[..., geo.pure_video_kv_start:geo.pure_video_kv_stop, :]
    k_t = k.transpose(-1, -2)
    pieces = []
    for start in range(0, q.shape[-2], q_chunk_tiles):
        stop = min(start + q_chunk_tiles, q.shape[-2])
        scores = torch.matmul(q[..., start:stop, :], k_t)
        pieces.append(torch.topk(scores, retained, dim=-1).indices)
    indices = pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim=-2)
    absolute = indices.to(torch.int32) + geo.pure_video_kv_start
    return absolute.sort(dim=-1).values


def context_tiles(geo):
    """KV tiles every query tile attends: all tiles that are not pure video."""
    before = torch.arange(0, geo.pure_video_kv_start, dtype=torch.int32)
    after = torch.arange(geo.pure_video_kv_stop, geo.kv_tiles, dtype=torch.int32)
    return torch.cat((before, after))


def compact_route(selected, geo):
    """Absolute ascending KV-tile list per pure-video query tile:
    ``context ++ selected`` merged in ascending order.  With video last this is
    triton_route.py:42-93 (context tiles all precede the video tiles)."""
    batch, heads, rows, _ = selected.shape
    before = torch.arange(0, geo.pure_video_kv_start, dtype=torch.int32)
    after = torch.arange(geo.pure_video_kv_stop, geo.kv_tiles, dtype=torch.int32)
    parts = []
    if before.numel():
        parts.append(before.view(1, 1, 1, -1).expand(batch, heads, rows, -1))
    parts.append(selected)
    if after.numel():
        parts.append(after.view(1, 1, 1, -1).expand(batch, heads, rows, -1))
    return torch.cat(parts, dim=-1).contiguous()


def delta_lut(selected, geo, batch, heads):
    """Delta-encoded LUT + valid counts.  router.py:219-240,453-531.
    ``selected`` None means fully dense.  Only defined for the reference-legal
    layout (video last)."""
    dense = torch.arange(geo.kv_tiles, dtype=torch.int32)
    dense_delta = torch.cat((dense[:1], dense[1:] - dense[:-1]))
    lut = dense_delta.view(1, 1, 1, -1).expand(batch, heads, geo.q_tiles, -1).clone()
    valid = torch.full((batch, heads, geo.q_tiles), geo.kv_tiles, dtype=torch.int32)
    if selected is None:
        return lut.contiguous(), valid.contiguous()
    if geo.pure_video_kv_stop != geo.kv_tiles or geo.pure_video_q_stop != geo.q_tiles:
        raise ValueError("delta LUT is only defined when video is the final segment")
    route = compact_route(selected, geo)
    delta = torch.cat((route[..., :1], route[..., 1:] - route[..., :-1]), dim=-1)
    lut[..., geo.pure_video_q_start:, : delta.shape[-1]] = delta
    valid[..., geo.pure_video_q_start:] = route.shape[-1]
    return lut.contiguous(), valid.contiguous()


def build_route(q, k, sequence, video_start, video_budget, video_stop=None):
    """Whole router from HND Q/K (router.py:248-275).  Returns
    ``(geo, retained, selected|None, route|None)``."""
    geo = geometry(sequence, video_start, video_stop)
    retained = retained_tiles(video_budget, geo)
    if retained == geo.pure_video_kv_tiles:
        return geo, retained, None, None
    selected = select_tiles(mean_pool(q, Q_TILE), mean_pool(k, KV_TILE), geo, retained)
    return geo, retained, selected, compact_route(selected, geo)


def route_row_lists(route, geo, head):
    """Python list of KV-tile lists, one per query tile, for one head."""
    rows = []
    everything = list(range(geo.kv_tiles))
    for tq in range(geo.q_tiles):
        if route is None or not (geo.pure_video_q_start <= tq < geo.pure_video_q_stop):
            rows.append(everything)
        else:
            rows.append(route[0, head, tq - geo.pure_video_q_start].tolist())
    return rows


# --------------------------------------------------------------------------
# Carriers
# --------------------------------------------------------------------------

def quantize_blocks(x, block, *, subtract_mean=False, mean=None):
    """Per-block INT8.  attention/sparse/sparse_sage.py:312-330.

    ``scale = amax|v|/127 + 1e-7``; ``code = trunc(v/scale +- 0.5)``.  With
    ``subtract_mean`` the per-(head,channel) mean over the whole sequence
    (taken in x.dtype, then widened) is removed first; ``mean`` overrides it."""
    b, h, sequence, dim = x.shape
    blocks = _ceil_div(sequence, block)
    output = torch.empty((b, h, sequence, dim), dtype=torch.int8)
    scales = torch.empty((b, h, blocks), dtype=torch.float32)
    if mean is None and subtract_mean:
        mean = x.mean(dim=-2, keepdim=True).float()
    elif mean is not None:
        mean = mean.reshape(b, h, 1, dim).float()
    for index in range(blocks):
        start, stop = index * block, min(index * block + block, sequence)
        value = x[..., start:stop, :].float()
        if mean is not None:
            value = value - mean
        scale = value.abs().amax(dim=(-2, -1)) / 127.0 + 1e-7
        quantized = value / scale[..., None, None]
        quantized = quantized + torch.where(quantized >= 0, 0.5, -0.5)
        output[..., start:stop, :].copy_(quantized.to(torch.int8))
        scales[..., index].copy_(scale)
    return output, scales


def block_summaries(x, block, dtype=None):
    """Tile means computed in FP32 and stored in ``dtype`` (default x.dtype).
    attention/sparse/chunked_qkv.py:102-116."""
    dtype = x.dtype if dtype is None else dtype
    return mean_pool(x.float(), block).to(dtype)


def v_fp8_carrier(v, bound=FP8_E4M3_MAX):
    """FP8-E4M3 V carrier ``(B,H,D,pad128(S))`` + scale ``(B,H,D)``.
    fp8_v_stream.py:50-75: ``scale = max(amax_s|v|/bound, 1e-20)``,
    ``code = e4m3(clamp(v/scale, +-bound))``, zero padding."""
    b, h, sequence, dim = v.shape
    padded = _ceil_div(sequence, 128) * 128
    amax = v.abs().amax(dim=2).to(torch.float32)
    scale = amax.div(float(bound)).clamp_min_(1.0e-20)
    value = v.float() / scale[:, :, None, :]
    value = value.clamp(-bound, bound).to(torch.float8_e4m3fn)
    carrier = torch.zeros((b, h, dim, padded), dtype=torch.float8_e4m3fn)
    carrier[..., :sequence] = value.transpose(-1, -2)
    return carrier, scale


# --------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------

def sparse_attention_int8_fp8(
    q8, q_scale, k8, k_scale, v_carrier, v_scale, geo, route,
    *, p_format="fp32", heads=None, q_tile_subset=None, out_dtype=torch.float32,
):
    """Block-sparse attention on the carriers.

    Per (head, query tile, listed KV tile), triton_sparse_kernels.py:164-197:
    ``logit2 = int32(q8 . k8) * q_scale[tq] * k_scale[tk] * D**-0.5 * log2(e)``,
    keys at positions >= S masked, softmax in FP32 with exp2, P @ V with V
    de-quantised from the FP8 carrier, ``out = acc / l``.

    ``p_format='fp32'`` keeps P in FP32 (the gate the tolerance is stated for).
    ``p_format='e4m3'`` rounds ``exp2(logit2 - ceil(rowmax) + 7)`` to FP8-E4M3
    before the product while the row sum stays FP32 - the arithmetic of the
    CUDA kernel's single-term mode.  ``p_format='e4m3x2'`` carries P as two
    E4M3 terms, ``hi`` = P truncated to 4 significant bits and ``lo`` =
    E4M3(P - hi) - the kernel's default; used as the tight implementation
    check."""
    _, h_total, sequence, dim = q8.shape
    heads = range(h_total) if heads is None else heads
    out = torch.zeros((1, h_total, sequence, dim), dtype=out_dtype)
    sm = dim ** -0.5 * LOG2E
    for head in heads:
        lists = route_row_lists(route, geo, head)
        k_i = k8[0, head].to(torch.float32)
        v_f = v_carrier[0, head, :, :].to(torch.float32)  # (D, padded)
        tiles = range(geo.q_tiles) if q_tile_subset is None else q_tile_subset
        for tq in tiles:
            q0, q1 = tq * Q_TILE, min(tq * Q_TILE + Q_TILE, sequence)
            blocks = lists[tq]
            pos = torch.cat([
                torch.arange(t * KV_TILE, min(t * KV_TILE + KV_TILE, sequence))
                for t in blocks
            ])
            tile_of = pos // KV_TILE
            s = q8[0, head, q0:q1].to(torch.float32) @ k_i[pos].T  # exact: |s| < 2^24
            logits = s * (q_scale[0, head, tq] * k_scale[0, head][tile_of] * sm)[None, :]
            row_max = logits.amax(dim=-1, keepdim=True)
            if p_format == "fp32":
                p = torch.exp2(logits - row_max)
                l = p.sum(dim=-1, keepdim=True)
            elif p_format == "e4m3":
                p = torch.exp2(logits - (torch.ceil(row_max) - P_EXPONENT_OFFSET))
                l = p.sum(dim=-1, keepdim=True)
                p = p.to(torch.float8_e4m3fn).to(torch.float32)
            elif p_format == "e4m3x2":
                p = torch.exp2(logits - (torch.ceil(row_max) - P_EXPONENT_OFFSET))
                l = p.sum(dim=-1, keepdim=True)
                hi = (p.view(torch.int32) & -0x00100000).view(torch.float32)
                lo = (p - hi).to(torch.float8_e4m3fn).to(torch.float32)
                p = hi.to(torch.float8_e4m3fn).to(torch.float32) + lo
            else:
                raise ValueError(p_format)
            acc = p @ v_f[:, pos].T
            acc = acc * v_scale[0, head][None, :] / l
            out[0, head, q0:q1] = acc.to(out_dtype)
    return out


def sparse_float_reference(q, k, v, geo, route, *, heads=None, q_tile_subset=None):
    """FP32 SDPA on the same block mask.  benchmarks/bench_sparse_backends.py:302-326."""
    _, h_total, sequence, dim = q.shape
    heads = range(h_total) if heads is None else heads
    out = torch.zeros((1, h_total, sequence, dim), dtype=torch.float32)
    scale = dim ** -0.5
    for head in heads:
        lists = route_row_lists(route, geo, head)
        tiles = range(geo.q_tiles) if q_tile_subset is None else q_tile_subset
        for tq in tiles:
            q0, q1 = tq * Q_TILE, min(tq * Q_TILE + Q_TILE, sequence)
            pos = torch.cat([
                torch.arange(t * KV_TILE, min(t * KV_TILE + KV_TILE, sequence))
                for t in lists[tq]
            ])
            q_rows = q[0, head, q0:q1].float()
            k_rows = k[0, head].index_select(0, pos).float()
            v_rows = v[0, head].index_select(0, pos).float()
            prob = torch.softmax(q_rows @ k_rows.T * scale, dim=-1)
            out[0, head, q0:q1] = prob @ v_rows
    return out


def compare(actual, reference):
    """cosine, relative max-abs, relative RMSE (bench_chunked_sparse_qkv.py:237-255)."""
    a = actual.double().flatten()
    r = reference.double().flatten()
    delta = a - r
    return dict(
        cosine=float((a @ r) / (a.norm() * r.norm()).clamp_min(1e-300)),
        rel_max_abs=float(delta.abs().max() / r.abs().max().clamp_min(1e-300)),
        rel_rmse=float(delta.norm() / r.norm().clamp_min(1e-300)),
        max_abs=float(delta.abs().max()),
    )


# --------------------------------------------------------------------------
# QKV projection (ConvRot INT8 GEMM)
# --------------------------------------------------------------------------

def hadamard(n):
    """Sylvester Hadamard matrix H_n (entries +-1), n a power of two."""
    h = torch.ones((1, 1), dtype=torch.float32)
    while h.shape[0] < n:
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    return h


def fwht_rows(x, group=256):
    """Unnormalised fast Walsh-Hadamard transform of every ``group``-wide slice
    of the last dimension, FP32, butterfly stages in ascending stride order
    (1, 2, 4, ... group/2): the lower element of a pair becomes a+b, the upper
    a-b.  Equals ``x @ hadamard(group)`` up to FP32 rounding; the CUDA prologue
    uses the same stage order, so the two agree bit for bit."""
    rows, channels = x.shape
    v = x.float().reshape(rows, channels // group, group)
    stride = 1
    while stride < group:
        w = v.reshape(rows, channels // group, group // (2 * stride), 2, stride)
        a, b = w[..., 0, :], w[..., 1, :]
        v = torch.stack((a + b, a - b), dim=-2).reshape(rows, channels // group, group)
        stride *= 2
    return v.reshape(rows, channels)


def convrot_quantize_rows(x, group=256):
    """Rotate each ``group``-channel slice of every row by the normalised
    Sylvester Hadamard ``H/sqrt(group)`` (FP32 FWHT), then per-row INT8:
    ``scale = amax/127`` (1 when the row is zero), ``code = rint(v/scale)``
    clamped to +-127.  Returns ``(codes int8 (S,C), scale fp32 (S,))``."""
    v = fwht_rows(x, group) * (1.0 / math.sqrt(group))
    amax = v.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    codes = torch.round(v / scale[:, None]).clamp_(-127, 127).to(torch.int8)
    return codes, scale


def qkv_project_int8(x_i8, x_scale, w_i8, w_scale, out_dtype=torch.bfloat16):
    """``y = bf16(float(int32 x.wT) * (x_scale[row] * w_scale[col]))``, the
    product of the two scales taken first (attention/sparse/fused_qkv.py:198-223,
    line 222).  Integer GEMM evaluated exactly in FP64 (|acc| <= 127*127*3072 < 2^53)."""
    acc = (x_i8.double() @ w_i8.double().T).to(torch.float32)
    y = acc * (x_scale[:, None] * w_scale[None, :])
    return y.to(out_dtype)


def rms_norm_rope_split_half(y, heads, q_norm, k_norm, epsilon, rope=None, head_dim=HEAD_DIM):
    """Per-head RMS norm and split-half rotation of the Q and K columns of a
    projected ``(S, 3*H*D)`` bf16 tensor; V columns pass through.  Follows the
    fused epilogue of the reference (attention/sparse/fused_qkv.py:225-289):

        v = bf16(y * rsqrt(sum_d y^2 / D + eps) * w[d])
        v[d], v[d+48] = bf16(f00*v[d] + f01*v[d+48]), bf16(f10*v[d] + f11*v[d+48])   d < 48

    with ``f = rope[0, s, 0, d]`` (2x2), every product and sum rounded to FP32.
    The sum of squares is taken in FP64 and rounded once, and the reciprocal
    square root is the correctly rounded one: the Triton kernel's reduction
    order and its approximate ``rsqrt`` are not pinned by any reference test
    (parity unpinned), so the restatement picks the order-free definition."""
    rows = y.shape[0]
    t = y.to(torch.bfloat16).float().reshape(rows, 3, heads, head_dim).clone()
    for kind, weight in ((0, q_norm), (1, k_norm)):
        x = t[:, kind]
        ss = (x.double() * x.double()).sum(dim=-1, keepdim=True).float()
        mean = ss * (1.0 / head_dim) + torch.tensor(float(epsilon), dtype=torch.float32)
        inverse_rms = (1.0 / mean.double().sqrt()).float()
        x = ((x * inverse_rms) * weight.float()).to(torch.bfloat16).float()
        if rope is not None:
            pairs = rope.shape[-3]
            f = rope.reshape(rows, 1, pairs, 2, 2).float()
            first, second = x[..., :pairs], x[..., pairs:2 * pairs]
            rotated_first = f[..., 0, 0] * first + f[..., 0, 1] * second
            rotated_second = f[..., 1, 0] * first + f[..., 1, 1] * second
            x = torch.cat([rotated_first, rotated_second, x[..., 2 * pairs:]], dim=-1).to(torch.bfloat16).float()
        t[:, kind] = x
    return t.reshape(rows, 3 * heads * head_dim).to(torch.bfloat16)


def make_rope(sequence):
    """The rotary table the reference's benchmarks use
    (benchmarks/bench_chunked_kitchen_qkv.py:193-204): bf16 (1,S,1,48,2,2)."""
    angles = torch.arange(sequence * 48, dtype=torch.float32).reshape(sequence, 48) * (1.0 / 8192.0)
    c, s = torch.cos(angles), torch.sin(angles)
    return torch.stack((c, -s, s, c), dim=-1).reshape(1, sequence, 1, 48, 2, 2).to(torch.bfloat16)


def split_heads_hnd(y, heads, head_dim=HEAD_DIM):
    """Columns ordered ``[Q heads | K heads | V heads]``, row
    ``kind*H*D + head*D + d`` (fused_qkv.py:195,394) -> three ``(1,H,S,D)``."""
    rows = y.shape[0]
    y = y.reshape(rows, 3, heads, head_dim).permute(1, 2, 0, 3)
    return y[0][None], y[1][None], y[2][None]
