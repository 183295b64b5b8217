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


class SymmetricHeadOutput:
    """Full ``(1, heads, S, 128)`` attention output living in symmetric memory,
    so that every rank can store its heads' tiles straight into every peer's
    copy (``ops.sparse_attention(..., peer_out_ptrs=...)``): the attention
    kernel then does the all-gather itself over NVLink and only a barrier is
    left.  Construction is collective.  Raises ``RuntimeError`` when symmetric
    memory is not available; callers then fall back to ``gather_heads``."""

    def __init__(self, heads, sequence, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.heads, self.sequence = int(heads), int(sequence)
        if self.world - 1 > 7:
            raise RuntimeError("at most 8 ranks can scatter to each other")
        numel = self.heads * self.sequence * 128
        self._flat = symm_mem.empty((numel,), dtype=dtype, device=device)
        self._handle = symm_mem.rendezvous(self._flat, self.group)
        self.tensor = self._flat.view(1, self.heads, self.sequence, 128)
        ptrs = [int(p) for p in self._handle.buffer_ptrs]
        if len(ptrs) != self.world or ptrs[self.rank] != self._flat.data_ptr():
            raise RuntimeError("symmetric memory rendezvous returned an unexpected pointer table")
        self._ptrs = ptrs
        self._head_bytes = self.sequence * 128 * self._flat.element_size()

    def local_slice(self):
        a, b = head_partition(self.heads, self.world, self.rank)
        return self.tensor[:, a:b]

    def peer_slice_ptrs(self):
        """Device addresses of this rank's head slice inside every peer's buffer."""
        a, _ = head_partition(self.heads, self.world, self.rank)
        return [p + a * self._head_bytes for r, p in enumerate(self._ptrs) if r != self.rank]

    def barrier(self):
        """Stream-ordered barrier across the ranks: once it has passed, every
        peer's stores into this rank's buffer (issued before their barrier) are
        visible here."""
        self._handle.barrier()
