"""Head sharding across the GPUs of one box.

Heads are independent end to end on this path (pooling, scores and top-k are
per head; scales are per (head, block); the attention kernel has no cross-head
term), so rank ``r`` owns the contiguous head range ``head_partition(H, W, r)``
and nothing crosses GPUs until the head-sharded output is reassembled.

``gather_heads`` reassembles with one NCCL all-gather over NVLink into a
``(1, H, S, 128)`` buffer (contiguous head ranges make the gathered layout the
HND tensor itself).  It also runs on the ``gloo`` backend, which is how the
CPU tests cover the N>1 host logic.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def head_partition(heads, world_size, rank):
    """Contiguous ``[start, stop)`` head range of ``rank``; the first
    ``heads % world_size`` ranks take one extra head."""
    heads, world_size, rank = int(heads), int(world_size), int(rank)
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank %d is outside world size %d" % (rank, world_size))
    if heads < world_size:
        raise ValueError("cannot shard %d heads over %d ranks" % (heads, world_size))
    base, extra = divmod(heads, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def gather_heads(local_out, heads, group=None, out=None):
    """All-gather head-sharded ``(1, h_local, S, 128)`` outputs into
    ``(1, heads, S, 128)``.  Every rank must hold the same number of heads
    (the uneven case falls back to a padded gather)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    _, h_local, sequence, dim = local_out.shape
    start, stop = head_partition(heads, world, rank)
    if stop - start != h_local:
        raise ValueError("rank %d holds %d heads, partition says %d" % (rank, h_local, stop - start))
    if out is None:
        out = torch.empty((1, heads, sequence, dim), dtype=local_out.dtype, device=local_out.device)
    local = local_out.contiguous()
    if heads % world == 0:
        dist.all_gather_into_tensor(out.view(heads, sequence, dim), local.view(h_local, sequence, dim), group=group)
        return out
    widest = -(-heads // world)
    padded = torch.zeros((widest, sequence, dim), dtype=local.dtype, device=local.device)
    padded[:h_local] = local[0]
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    for r, piece in enumerate(pieces):
        a, b = head_partition(heads, world, r)
        out[0, a:b] = piece[: b - a]
    return out
