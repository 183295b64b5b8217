"""Import the reference's own modules from ``oracle/_ref``.  TEST INFRASTRUCTURE ONLY.

``oracle/build_ref.py`` stages the unmodified ``h3_optimizations`` package and
``benchmarks`` directory of Pizzawookiee/H3-Optimizations there.  This module
makes them importable and hands out the handful of functions the checker and
the timed CPU baseline use.  The product package never imports it.
"""

from __future__ import annotations

import importlib
import sys
from pathlib import Path
from types import SimpleNamespace

REF_ROOT = Path(__file__).resolve().parent / "_ref"


class ReferenceUnavailable(RuntimeError):
    pass


def available():
    return (REF_ROOT / "h3_optimizations" / "attention" / "sparse" / "router.py").exists()


def _ensure_path():
    if not available():
        raise ReferenceUnavailable(
            "oracle/_ref is empty: run `python oracle/build_ref.py --reference <checkout>` where the "
            "reference is checked out (it ships to the GPU box with the repository snapshot)"
        )
    for entry in (str(REF_ROOT / "benchmarks"), str(REF_ROOT)):
        if entry not in sys.path:
            sys.path.insert(0, entry)


def module(name):
    """``importlib.import_module`` of a staged reference module, e.g.
    ``h3_optimizations.attention.sparse.router`` or ``bench_sparse_backends``."""
    _ensure_path()
    loaded = importlib.import_module(name)
    origin = Path(getattr(loaded, "__file__", "") or "").resolve()
    if REF_ROOT.resolve() not in origin.parents:
        raise ReferenceUnavailable("%s resolved to %s, not to the staged reference" % (name, origin))
    return loaded


def router_module():
    return module("h3_optimizations.attention.sparse.router")


def bench_module():
    """benchmarks/bench_sparse_backends.py (sparse_float_reference, absolute_lut)."""
    return module("bench_sparse_backends")


def triton_kernels_module():
    """attention/sparse/triton_sparse_kernels.py; needs Triton and a GPU to launch."""
    return module("h3_optimizations.attention.sparse.triton_sparse_kernels")


def layout(sequence, segments, video_range, video_shape=None, audio_t=0):
    """The attributes the reference router reads from a packed layout
    (attention/sparse/router.py:111-122)."""
    video_range = (int(video_range[0]), int(video_range[1]))
    if video_shape is None:
        video_shape = (1, 1, video_range[1] - video_range[0])
    return SimpleNamespace(seq_len=int(sequence), video_range=video_range, segments=tuple(segments),
                           video_shape=tuple(video_shape), audio_t=int(audio_t))


def build_lut(q, k, sequence, video_start, budget, segments=None):
    """``SparseTileRouter.build_lut`` (attention/sparse/router.py:248) on HND
    Q/K with the video segment last.  Returns ``(lut, valid, metadata)``."""
    router = router_module().SparseTileRouter(q_tile=128, kv_tile=64)
    if segments is None:
        segments = ((0, int(video_start), "text"), (int(video_start), int(sequence), "video"))
        if video_start == 0:
            segments = segments[1:]
    return router.build_lut(q, k, layout(sequence, segments, (video_start, sequence)), budget)


def sparse_float_reference(q, k, v, lut, valid):
    """benchmarks/bench_sparse_backends.py:302-326: FP32 SDPA on the LUT's block mask."""
    import torch

    return bench_module().sparse_float_reference(torch, q, k, v, lut, valid, 128, 64)
