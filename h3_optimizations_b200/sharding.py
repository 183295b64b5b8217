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


def shard_qkv_weight(weight, scale, heads, start, stop, head_dim=128):
    """Rows of a fused QKV weight ``(3*heads*head_dim, hidden)`` (and of its
    per-row scale) that produce heads ``[start, stop)``: the Q, K and V rows of
    those heads, kept in the ``[Q heads | K heads | V heads]`` order the
    projection expects (row ``kind*H*D + head*D + d``, fused_qkv.py:195,394).
    A rank that projects with this slice and ``heads = stop - start`` emits the
    carriers of exactly its own heads; the activations are replicated."""
    heads, start, stop = int(heads), int(start), int(stop)
    if not 0 <= start < stop <= heads:
        raise ValueError("head range [%d, %d) is outside %d heads" % (start, stop, heads))
    if weight.shape[0] != 3 * heads * head_dim or scale.shape[0] != weight.shape[0]:
        raise ValueError("weight rows %d do not match 3 * %d heads * %d" % (weight.shape[0], heads, head_dim))
    rows = torch.cat([
        torch.arange((kind * heads + start) * head_dim, (kind * heads + stop) * head_dim, device=weight.device)
        for kind in range(3)
    ])
    return weight.index_select(0, rows).contiguous(), scale.index_select(0, rows).contiguous()


class HeadShardedBackend:
    """One rank of a head-sharded attention layer (one process per GPU).

    Wraps a ``B200SparseBackend`` that owns the contiguous head range
    ``head_partition(heads, world, rank)``.  ``prepare`` / ``prepare_projected``
    work on the local heads and involve no communication.  ``execute`` launches
    the attention kernel and reassembles the ``(1, heads, S, 128)`` output on
    every rank:

    * ``exchange="peer"``: the output lives in symmetric memory and the kernel
      stores every finished tile into all peers' copies itself (plain stores
      over NVLink); a stream-ordered barrier closes the step.
    * ``exchange="nccl"``: one NCCL all-gather after the kernel.
    * ``exchange="auto"`` (default): ``peer`` when every rank can set it up,
      agreed with one all-reduce at the first ``execute``; ``nccl`` otherwise.

    ``forward_host`` is the host-resident entry of the local heads: every rank
    streams its own Q/K/V slice in and its own output slice out over its own
    PCIe link (``B200SparseBackend.forward_host``); nothing crosses GPUs.
    """

    def __init__(self, backend, heads, *, group=None, exchange="auto"):
        if exchange not in ("auto", "peer", "nccl"):
            raise ValueError("exchange must be 'auto', 'peer' or 'nccl'")
        self.backend = backend
        self.heads = int(heads)
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.head_range = head_partition(self.heads, self.world, self.rank)
        self.requested_exchange = exchange
        self.exchange = None          # decided at the first execute
        self.exchange_note = ""
        self._symmetric = None
        self._peer_ptrs = None
        self._full = None
        self._key = None

    @property
    def local_heads(self):
        return self.head_range[1] - self.head_range[0]

    def prepare(self, q, k, v, *, layer_index, transformer_options):
        if q.shape[1] != self.local_heads:
            raise ValueError("rank %d owns %d heads, got %d" % (self.rank, self.local_heads, q.shape[1]))
        return self.backend.prepare(q, k, v, layer_index=layer_index, transformer_options=transformer_options)

    def prepare_projected(self, projected, *, layer_index, transformer_options):
        if int(projected.heads) != self.local_heads:
            raise ValueError("rank %d owns %d heads, got %d" % (self.rank, self.local_heads, projected.heads))
        return self.backend.prepare_projected(projected, layer_index=layer_index, transformer_options=transformer_options)

    def _setup(self, sequence, dtype, device):
        key = (int(sequence), dtype, device)
        if self._key == key:
            return
        self._symmetric = self._peer_ptrs = self._full = None
        failure = None
        if self.requested_exchange in ("auto", "peer"):
            try:
                self._symmetric = SymmetricHeadOutput(self.heads, sequence, dtype, device, self.group)
                self._peer_ptrs = self._symmetric.peer_slice_ptrs()
            except Exception as exc:  # symmetric memory unavailable on this rank
                self._symmetric, failure = None, exc
        # every rank must take the same path
        agreed = torch.tensor([1 if self._symmetric is not None else 0], dtype=torch.int32, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.group)
        if int(agreed.item()) == 1:
            self.exchange = "peer"
            self.exchange_note = "attention epilogue stores every tile into all peers' buffers (P2P over NVLink) + barrier"
            self._full = self._symmetric.tensor
        else:
            if self.requested_exchange == "peer":
                raise RuntimeError("peer exchange requested but symmetric memory is unavailable: %s"
                                   % (failure if failure is not None else "a peer could not set it up"))
            reason = "requested" if self.requested_exchange == "nccl" else str(
                failure if failure is not None else "a peer could not set up symmetric memory").splitlines()[0][:80]
            self._symmetric = self._peer_ptrs = None
            self.exchange = "nccl"
            self.exchange_note = "NCCL all-gather after the kernel (%s)" % reason
            self._full = torch.empty((1, self.heads, int(sequence), 128), dtype=dtype, device=device)
        self._key = key

    def execute(self, prepared, kernel_done=None):
        """Attention on the local heads + reassembly.  Returns the full
        ``(1, heads, S, 128)`` output (the same buffer on every call).
        ``kernel_done``: optional CUDA event recorded between the attention
        kernel and the reassembly step (benchmarks time the two apart)."""
        sparse = prepared.sparse
        self._setup(sparse.sequence, sparse.output_dtype, sparse.q_int8.device)
        a, b = self.head_range
        local = self._full[:, a:b]
        if self.exchange == "peer":
            self.backend.execute(prepared, out=local, peer_out_ptrs=self._peer_ptrs)
            if kernel_done is not None:
                kernel_done.record()
            self._symmetric.barrier()
        else:
            self.backend.execute(prepared, out=local)
            if kernel_done is not None:
                kernel_done.record()
            # the local slice is part of the gathered buffer: the collective reads a copy of it
            gather_heads(local.clone(), self.heads, self.group, out=self._full)
        return self._full

    def capture(self, q, k, v, *, layer_index, transformer_options):
        """Local prepare + attention + exchange as a replayable CUDA graph
        (``backend.CapturedLayerCall``).  Collective: every rank captures, and
        every rank replays the same number of times."""
        from .backend import CapturedLayerCall

        if self.exchange is None:  # the ranks agree on the exchange path at the first call
            self.execute(self.prepare(q, k, v, layer_index=layer_index, transformer_options=transformer_options))
        if self.exchange != "peer":
            raise RuntimeError("only the peer-store exchange is captured; with the NCCL all-gather run the step eagerly")
        return CapturedLayerCall(self, q, k, v, layer_index=layer_index, transformer_options=transformer_options)

    def check_exchange(self, prepared):
        """Collective self-check: the reassembled output must equal an NCCL
        all-gather of the local slices bit for bit.  Returns True/False."""
        full = self.execute(prepared)
        if full.is_cuda:
            torch.cuda.synchronize(full.device)
        a, b = self.head_range
        expected = gather_heads(full[:, a:b].clone(), self.heads, self.group)
        if full.is_cuda:
            torch.cuda.synchronize(full.device)
        same = torch.tensor([1 if torch.equal(expected, full) else 0], dtype=torch.int32, device=full.device)
        dist.all_reduce(same, op=dist.ReduceOp.MIN, group=self.group)
        return bool(int(same.item()))

    def forward_host(self, q, k, v, out=None, *, layer_index, transformer_options, heads_per_chunk=None):
        """Host-resident entry of this rank's heads: Q/K/V ``(1, h_local, S, 128)``
        in (pinned) host memory in, the matching output slice out, copies and
        kernels pipelined over three streams.  No exchange: across the ranks the
        layer's output arrives in host memory over all their PCIe links at once."""
        if q.shape[1] != self.local_heads:
            raise ValueError("rank %d owns %d heads, got %d" % (self.rank, self.local_heads, q.shape[1]))
        return self.backend.forward_host(q, k, v, out, layer_index=layer_index,
                                         transformer_options=transformer_options, heads_per_chunk=heads_per_chunk)
