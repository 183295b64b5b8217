"""Shared test helpers (input checksums, mask decoding)."""

import hashlib
from types import SimpleNamespace

import numpy as np
import torch


def checksum(*tensors):
    digest = hashlib.sha256()
    for t in tensors:
        digest.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return digest.hexdigest()


def layout_of(sequence, video_start, video_stop=None):
    video_stop = sequence if video_stop is None else video_stop
    segments = [(0, video_start, "text"), (video_start, video_stop, "video")]
    if video_stop < sequence:
        segments.append((video_stop, sequence, "text"))
    if video_start == 0:
        segments = segments[1:]
    return SimpleNamespace(
        seq_len=sequence,
        video_range=(video_start, video_stop),
        segments=tuple(segments),
        video_shape=(1, 1, video_stop - video_start),
        audio_t=0,
    )


def mask_from_route(route, geo, heads):
    """Boolean (H,Tq,Tk) block mask from a packed route (None = dense)."""
    mask = torch.ones((heads, geo.q_tiles, geo.kv_tiles), dtype=torch.bool)
    if route is None:
        return mask
    rows = torch.zeros((heads, route.shape[2], geo.kv_tiles), dtype=torch.bool)
    rows.scatter_(2, route[0].long().cpu(), True)
    mask[:, geo.pure_video_q_start:geo.pure_video_q_stop] = rows
    return mask


def mask_from_bits(bits, kv_tiles):
    return torch.from_numpy(np.unpackbits(bits, axis=-1)[..., :kv_tiles].astype(bool))


def mask_from_lut(lut, valid):
    absolute = torch.cumsum(lut[0], dim=-1)
    heads, q_tiles, kv_tiles = absolute.shape
    live = torch.arange(kv_tiles)[None, None, :] < valid[0][..., None]
    hits = torch.zeros((heads, q_tiles, kv_tiles), dtype=torch.int32)
    hits.scatter_add_(2, absolute.clamp(0, kv_tiles - 1).long(), live.to(torch.int32))
    mask = hits > 0
    return mask
