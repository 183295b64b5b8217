"""Seeded synthetic inputs for the benchmark configurations.

No dataset or checkpoint is involved anywhere on this path; every input is
drawn from a CPU ``torch.Generator`` so that the CPU checker and the GPU see
identical bits.  Shapes and distributions:

* ``config0``: B1 H4 D128, 256 text + 2048 video tokens (video is the final
  segment, the only order the reference router accepts,
  attention/sparse/router.py:133-138); Q/K/V ~ N(0,1) drawn in bf16 and
  widened to fp32.
* ``config1``: B1 H24 D128, 512 text + 32760 video tokens (21x30x52 latent
  grid, row-major); Q and K are ``N(0,1) + Z @ U`` with a per-head rank-8
  basis ``U ~ N(0,1)`` (8x128) and coefficients ``Z ~ N(0, 0.5^2)`` held
  constant over each 64-token group so that tile means carry signal; V is
  plain N(0,1); bf16.
* ``config3``: as config1 with 512 text + 75600 video tokens (21x60x60).
* ``config2_projection``: activations (S,3072) bf16 N(0,1), INT8 weight
  (9216,3072) uniform in [-127,127], per-row scale 1/(127*sqrt(3072)).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from types import SimpleNamespace

import torch

HEAD_DIM = 128


@dataclass(frozen=True)
class SequenceSpec:
    name: str
    heads: int
    segments: tuple  # ((start, stop, kind), ...)
    video_shape: tuple
    audio_t: int = 0

    @property
    def sequence(self):
        return self.segments[-1][1]

    @property
    def video_range(self):
        for start, stop, kind in self.segments:
            if kind == "video":
                return (start, stop)
        raise ValueError("no video segment")

    def layout(self):
        """Duck-typed packed layout with the fields the router reads
        (router.py:111-122)."""
        return SimpleNamespace(
            seq_len=self.sequence,
            video_range=self.video_range,
            segments=tuple(self.segments),
            video_shape=tuple(self.video_shape),
            audio_t=int(self.audio_t),
        )


def _segments(*pairs):
    out, cursor = [], 0
    for kind, length in pairs:
        out.append((cursor, cursor + length, kind))
        cursor += length
    return tuple(out)


CONFIG0 = SequenceSpec("config0", 4, _segments(("text", 256), ("video", 2048)), (1, 32, 64))
CONFIG1 = SequenceSpec("config1", 24, _segments(("text", 512), ("video", 32760)), (21, 30, 52))
CONFIG3 = SequenceSpec("config3", 24, _segments(("text", 512), ("video", 75600)), (21, 60, 60))
CONFIG4 = SequenceSpec(
    "config4", 24,
    _segments(("text", 512), ("ref_img", 1024), ("audio", 1536), ("video", 32760)),
    (21, 30, 52), audio_t=768,
)
# Video first, text after it (the order the benchmark description words it in); the reference router rejects
# it, the generalised router here accepts it.
CONFIG0_VIDEO_FIRST = SequenceSpec(
    "config0_video_first", 4, _segments(("video", 2048), ("text", 256)), (1, 32, 64)
)


def small_spec(name, heads, context, video, *, kinds=("text",)):
    """Arbitrary small layout for tests: ``context`` tokens split evenly over
    ``kinds`` followed by ``video`` tokens."""
    pairs = []
    per = context // max(1, len(kinds))
    left = context
    for index, kind in enumerate(kinds):
        length = left if index == len(kinds) - 1 else per
        if length:
            pairs.append((kind, length))
        left -= length
    pairs.append(("video", video))
    return SequenceSpec(name, heads, _segments(*pairs), (1, 1, video))


def gaussian_qkv(spec, seed=0, dtype=torch.bfloat16, widen=False):
    """config0-style inputs: i.i.d. N(0,1) drawn in ``dtype``."""
    gen = torch.Generator().manual_seed(seed)
    shape = (1, spec.heads, spec.sequence, HEAD_DIM)
    out = []
    for _ in range(3):
        t = torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)
        out.append(t.float() if widen else t)
    return tuple(out)


def structured_qkv(spec, seed=0, dtype=torch.bfloat16, rank=8, coeff_std=0.5, group=64,
                   heads=None):
    """config1-style inputs (rank-8 structure on Q and K, plain V).

    Each head draws from its own generator stream (``seed*1000003 + head``) so
    a head subset reproduces the full tensor's values for those heads."""
    heads = list(range(spec.heads)) if heads is None else list(heads)
    sequence = spec.sequence
    groups = (sequence + group - 1) // group
    q = torch.empty((1, len(heads), sequence, HEAD_DIM), dtype=dtype)
    k = torch.empty_like(q)
    v = torch.empty_like(q)
    for slot, head in enumerate(heads):
        gen = torch.Generator().manual_seed(seed * 1000003 + head)
        for dst in (q, k):
            noise = torch.randn((sequence, HEAD_DIM), generator=gen)
            basis = torch.randn((rank, HEAD_DIM), generator=gen)
            coeff = torch.randn((groups, rank), generator=gen) * coeff_std
            low = (coeff @ basis).repeat_interleave(group, dim=0)[:sequence]
            dst[0, slot] = (noise + low).to(dtype)
        v[0, slot] = torch.randn((sequence, HEAD_DIM), generator=gen).to(dtype)
    return q, k, v


def projection_inputs(sequence, hidden=3072, heads=24, seed=0):
    """config2 projection operands: ``x`` bf16 (S,hidden), ``w`` int8
    (3*heads*128, hidden), ``w_scale`` fp32 (3*heads*128,)."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn((sequence, hidden), generator=gen).to(torch.bfloat16)
    out_features = 3 * heads * HEAD_DIM
    w = torch.randint(-127, 128, (out_features, hidden), generator=gen, dtype=torch.int16).to(torch.int8)
    w_scale = torch.full((out_features,), 1.0 / (127.0 * math.sqrt(hidden)), dtype=torch.float32)
    return x, w, w_scale


def attention_pair_count(geo, retained):
    """(q-tile, kv-tile) pairs the kernel visits, per head."""
    dense_rows = geo.q_tiles - geo.pure_video_q_tiles
    if retained >= geo.pure_video_kv_tiles:
        return geo.q_tiles * geo.kv_tiles
    return dense_rows * geo.kv_tiles + geo.pure_video_q_tiles * (geo.context_kv_tiles + retained)
