"""Fixed-density tile router (host side) for the B200 sparse backend.

Keeps the surface of the reference router (attention/sparse/router.py):
``geometry`` / ``build_lut`` / ``build_lut_from_summaries`` with the same
argument meaning, metadata and errors, and adds ``build_route*`` which return
the packed absolute block-index list the attention kernel consumes directly
(the reference's "compact absolute" encoding, attention/sparse/triton_route.py:42-93).

Two deliberate differences, both stated where they apply:

* the video segment need not be the final one: a tile is routed sparsely only
  when it lies entirely inside the video range, every other tile (text, audio,
  reference conditioning, tiles straddling a boundary) stays dense.  With the
  video last this is exactly the reference rule; ``require_video_last=True``
  restores the reference's rejection of other layouts.
* scores are exact FP64 dot products of the tile means and equal scores keep
  the lower tile index; the reference scores in the input dtype and leaves tie
  order to ``torch.topk``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import ops
from .config import DENSITY_FIXED
from .errors import SparseRouterError

Q_TILE = 128
KV_TILE = 64


@dataclass(frozen=True)
class SparseTileGeometry:
    signature: tuple
    sequence: int
    q_tiles: int
    kv_tiles: int
    pure_video_q_start: int
    pure_video_kv_start: int
    pure_video_q_stop: int = -1
    pure_video_kv_stop: int = -1

    def __post_init__(self):
        if self.pure_video_q_stop < 0:
            object.__setattr__(self, "pure_video_q_stop", self.q_tiles)
        if self.pure_video_kv_stop < 0:
            object.__setattr__(self, "pure_video_kv_stop", self.kv_tiles)

    @property
    def pure_video_q_tiles(self):
        return self.pure_video_q_stop - self.pure_video_q_start

    @property
    def pure_video_kv_tiles(self):
        return self.pure_video_kv_stop - self.pure_video_kv_start

    @property
    def context_kv_tiles(self):
        return self.kv_tiles - self.pure_video_kv_tiles


@dataclass(frozen=True)
class SparseMaskMetadata:
    requested_video_budget: float
    actual_video_tile_density: float
    full_mask_density: float
    dense_q_tiles: int
    sparse_q_tiles: int
    q_tiles: int
    kv_tiles: int
    pure_video_q_tiles: int
    pure_video_kv_tiles: int
    retained_video_kv_tiles: int
    density_mode: str = DENSITY_FIXED

    def as_dict(self):
        return dict(vars(self))


@dataclass
class SparseRoute:
    """Packed route: ``indices`` int32 ``(1,H,pure_q,route_len)`` ascending
    absolute KV tiles for the pure-video query tiles, or None when dense."""

    indices: torch.Tensor | None
    geometry: SparseTileGeometry
    retained: int
    metadata: SparseMaskMetadata

    @property
    def route_len(self):
        return 0 if self.indices is None else int(self.indices.shape[-1])


class SparseTileRouter:
    def __init__(self, config=None, *, spec=None, q_tile=None, kv_tile=None, require_video_last=False):
        self.config = config
        self.spec = spec
        self.q_tile = int(q_tile if q_tile is not None else getattr(spec, "q_tile", Q_TILE))
        self.kv_tile = int(kv_tile if kv_tile is not None else getattr(spec, "kv_tile", KV_TILE))
        if self.q_tile <= 0 or self.kv_tile <= 0:
            raise ValueError("Sparse Sage tile sizes must be positive")
        if (self.q_tile, self.kv_tile) != (Q_TILE, KV_TILE):
            raise ValueError("the B200 kernels are built for 128-row query and 64-row KV tiles")
        self.require_video_last = bool(require_video_last)
        self._geometry_cache = {}

    # -- host geometry (reference: router.py:111-217) ---------------------

    @staticmethod
    def _layout_signature(layout):
        return (
            int(layout.seq_len),
            tuple(int(x) for x in layout.video_range),
            tuple((int(a), int(b), str(kind)) for a, b, kind in layout.segments),
            tuple(int(x) for x in layout.video_shape),
            int(layout.audio_t),
        )

    def geometry(self, layout):
        signature = self._layout_signature(layout)
        cached = self._geometry_cache.get(signature)
        if cached is not None:
            return cached
        sequence = int(layout.seq_len)
        video_start, video_stop = (int(x) for x in layout.video_range)
        if sequence <= 0:
            raise SparseRouterError("packed sequence is empty")
        legal = 0 <= video_start < video_stop <= sequence
        if self.require_video_last:
            legal = legal and video_stop == sequence
        if not legal:
            raise SparseRouterError(
                "Sparse Sage requires target video to be the final packed "
                "segment; got video=%s sequence=%d" % (tuple(layout.video_range), sequence)
            )
        q_tiles = (sequence + self.q_tile - 1) // self.q_tile
        kv_tiles = (sequence + self.kv_tile - 1) // self.kv_tile
        last = video_stop == sequence
        geometry = SparseTileGeometry(
            signature=signature,
            sequence=sequence,
            q_tiles=q_tiles,
            kv_tiles=kv_tiles,
            pure_video_q_start=(video_start + self.q_tile - 1) // self.q_tile,
            pure_video_kv_start=(video_start + self.kv_tile - 1) // self.kv_tile,
            pure_video_q_stop=q_tiles if last else video_stop // self.q_tile,
            pure_video_kv_stop=kv_tiles if last else video_stop // self.kv_tile,
        )
        if geometry.pure_video_q_tiles <= 0:
            raise SparseRouterError("packed layout has no pure-video query tiles")
        if geometry.pure_video_kv_tiles <= 0:
            raise SparseRouterError("packed layout has no pure-video KV tiles")
        self._geometry_cache[signature] = geometry
        return geometry

    @staticmethod
    def _retained(video_budget, geometry):
        # host double arithmetic on purpose: budget*tiles products within one
        # ulp of an integer must round as Python does
        return min(
            geometry.pure_video_kv_tiles,
            max(1, int(math.ceil(float(video_budget) * geometry.pure_video_kv_tiles))),
        )

    @staticmethod
    def _metadata(geometry, video_budget, retained):
        pure_q = geometry.pure_video_q_tiles
        pure_kv = geometry.pure_video_kv_tiles
        sparse_q = pure_q if retained < pure_kv else 0
        non_video_kv = geometry.kv_tiles - pure_kv
        true_blocks = (geometry.q_tiles - pure_q) * geometry.kv_tiles + pure_q * (non_video_kv + retained)
        return SparseMaskMetadata(
            requested_video_budget=float(video_budget),
            actual_video_tile_density=float(retained) / pure_kv,
            full_mask_density=float(true_blocks) / (geometry.q_tiles * geometry.kv_tiles),
            dense_q_tiles=geometry.q_tiles - sparse_q,
            sparse_q_tiles=sparse_q,
            q_tiles=geometry.q_tiles,
            kv_tiles=geometry.kv_tiles,
            pure_video_q_tiles=pure_q,
            pure_video_kv_tiles=pure_kv,
            retained_video_kv_tiles=retained,
        )

    @staticmethod
    def _check_budget(video_budget):
        if not 0.01 <= float(video_budget) <= 1.0:
            raise SparseRouterError("video_budget must be in [0.01, 1]")

    def _notify(self, sink, geometry, route):
        """``sink(indices|None, geometry, kv_tile)`` with pure-video-relative
        tile indices (router.py:242-246); here they arrive sorted ascending
        rather than in top-k order, which the histogram consumer ignores."""
        if sink is None:
            return
        if route is None:
            sink(None, geometry, self.kv_tile)
            return
        start = geometry.pure_video_kv_start
        selected = route[..., start:start + (route.shape[-1] - geometry.context_kv_tiles)]
        sink(selected.to(torch.int64) - start, geometry, self.kv_tile)

    # -- packed routes (what the kernel consumes) ---------------------------

    def build_route_from_summaries(self, q_summary, k_summary, layout, video_budget, *, sink=None):
        if q_summary.ndim != 4 or k_summary.ndim != 4:
            raise SparseRouterError("tile router summaries must be rank-4 HND tensors")
        if q_summary.shape[:2] != k_summary.shape[:2]:
            raise SparseRouterError("Q/K router summary batch and head shapes differ")
        if q_summary.shape[-1] != k_summary.shape[-1]:
            raise SparseRouterError("Q/K router summary dimensions differ")
        if q_summary.device != k_summary.device:
            raise SparseRouterError("Q/K router summary devices differ")
        self._check_budget(video_budget)
        geometry = self.geometry(layout)
        expected_q = (geometry.q_tiles, q_summary.shape[-1])
        expected_k = (geometry.kv_tiles, k_summary.shape[-1])
        if tuple(q_summary.shape[-2:]) != expected_q:
            raise SparseRouterError(
                "Q router summary shape %s does not match %s" % (tuple(q_summary.shape[-2:]), expected_q)
            )
        if tuple(k_summary.shape[-2:]) != expected_k:
            raise SparseRouterError(
                "K router summary shape %s does not match %s" % (tuple(k_summary.shape[-2:]), expected_k)
            )
        retained = self._retained(video_budget, geometry)
        metadata = self._metadata(geometry, video_budget, retained)
        if retained == geometry.pure_video_kv_tiles:
            self._notify(sink, geometry, None)
            return SparseRoute(None, geometry, retained, metadata)
        if q_summary.shape[0] != 1:
            raise SparseRouterError("released H3 expects attention batch 1")
        indices = ops.route_topk(
            q_summary, k_summary,
            q_start=geometry.pure_video_q_start, q_stop=geometry.pure_video_q_stop,
            kv_start=geometry.pure_video_kv_start, kv_stop=geometry.pure_video_kv_stop,
            retained=retained,
        )
        self._notify(sink, geometry, indices)
        return SparseRoute(indices, geometry, retained, metadata)

    def build_route(self, q, k, layout, video_budget, *, sink=None):
        if q.ndim != 4 or k.ndim != 4:
            raise SparseRouterError("tile router expects HND rank-4 Q/K")
        if q.shape != k.shape:
            raise SparseRouterError(
                "tile router requires equal Q/K shapes; got %s %s" % (tuple(q.shape), tuple(k.shape))
            )
        self._check_budget(video_budget)
        geometry = self.geometry(layout)
        if q.shape[-2] != geometry.sequence:
            raise SparseRouterError(
                "layout sequence %d does not match Q/K sequence %d" % (geometry.sequence, q.shape[-2])
            )
        retained = self._retained(video_budget, geometry)
        if retained == geometry.pure_video_kv_tiles:
            # full budget: no pooling, no scoring (router.py:266-268)
            self._notify(sink, geometry, None)
            return SparseRoute(None, geometry, retained, self._metadata(geometry, video_budget, retained))
        q_summary = ops.tile_means(q, self.q_tile)
        k_summary = ops.tile_means(k, self.kv_tile)
        return self.build_route_from_summaries(q_summary, k_summary, layout, video_budget, sink=sink)

    # -- reference-format outputs ---------------------------------------------

    def _lut(self, route, device, heads):
        geometry = route.geometry
        if route.indices is not None and (
            geometry.pure_video_kv_stop != geometry.kv_tiles or geometry.pure_video_q_stop != geometry.q_tiles
        ):
            raise SparseRouterError("the delta LUT encoding is only defined when video is the final segment")
        lut, valid = ops.route_to_delta_lut(
            route.indices, heads=heads, q_tiles=geometry.q_tiles, kv_tiles=geometry.kv_tiles,
            q_start=geometry.pure_video_q_start, q_stop=geometry.pure_video_q_stop, device=device,
        )
        return lut, valid, route.metadata

    def build_lut(self, q, k, layout, video_budget, *, sink=None):
        """``(lut int32 (1,H,Tq,Tk) delta-encoded, valid int32 (1,H,Tq), metadata)``."""
        route = self.build_route(q, k, layout, video_budget, sink=sink)
        return self._lut(route, q.device, q.shape[1])

    def build_lut_from_summaries(self, q_summary, k_summary, layout, video_budget, *, sink=None):
        route = self.build_route_from_summaries(q_summary, k_summary, layout, video_budget, sink=sink)
        return self._lut(route, q_summary.device, q_summary.shape[1])
