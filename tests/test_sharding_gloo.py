"""Head sharding host logic with two CPU ranks (gloo); no GPU."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from h3_optimizations_b200.sharding import gather_heads, head_partition


def test_head_partition_is_contiguous_and_complete():
    for heads, world in ((24, 1), (24, 2), (24, 4), (24, 8), (7, 3), (5, 5)):
        ranges = [head_partition(heads, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == heads
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        sizes = [b - a for a, b in ranges]
        assert max(sizes) - min(sizes) <= 1
    assert [head_partition(24, 8, r) for r in (0, 7)] == [(0, 3), (21, 24)]
    with pytest.raises(ValueError):
        head_partition(2, 4, 0)
    with pytest.raises(ValueError):
        head_partition(8, 4, 4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, heads, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sequence = 37
        full = torch.arange(heads * sequence * 128, dtype=torch.float32).reshape(1, heads, sequence, 128)
        a, b = head_partition(heads, world, rank)
        gathered = gather_heads(full[:, a:b].clone(), heads)
        ok = torch.equal(gathered, full)
        # in-place form used by the benchmark: the local slice already sits in the output buffer
        buffer = torch.zeros_like(full)
        buffer[:, a:b] = full[:, a:b]
        if heads % world == 0:
            ok = ok and torch.equal(gather_heads(buffer[:, a:b], heads, out=buffer), full)
        bad = False
        try:
            gather_heads(full[:, : (b - a) + 1], heads)
        except ValueError:
            bad = True
        queue.put((rank, ok and bad))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("heads", [4, 5])
def test_gather_heads_two_gloo_ranks(heads):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, heads, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def test_shard_qkv_weight_keeps_kind_major_order():
    from h3_optimizations_b200.sharding import shard_qkv_weight

    heads, hidden = 4, 8
    weight = torch.arange(3 * heads * 128 * hidden, dtype=torch.int32).reshape(3 * heads * 128, hidden)
    scale = torch.arange(3 * heads * 128, dtype=torch.float32)
    w, s = shard_qkv_weight(weight, scale, heads, 1, 3)
    assert tuple(w.shape) == (3 * 2 * 128, hidden)
    for kind in range(3):
        rows = slice(kind * 2 * 128, (kind + 1) * 2 * 128)
        source = slice((kind * heads + 1) * 128, (kind * heads + 3) * 128)
        assert torch.equal(w[rows], weight[source]) and torch.equal(s[rows], scale[source])
    with pytest.raises(ValueError):
        shard_qkv_weight(weight, scale, heads, 2, 5)


class _StubBackend:
    """Stands in for B200SparseBackend on the CPU: `execute` fills its slice of
    the output with values that identify (head, row)."""

    def __init__(self, first_head):
        self.first_head = first_head

    def prepare(self, q, k, v, *, layer_index, transformer_options):
        from types import SimpleNamespace

        sparse = SimpleNamespace(sequence=q.shape[2], output_dtype=q.dtype, q_int8=q, heads=q.shape[1])
        return SimpleNamespace(sparse=sparse)

    def execute(self, prepared, out=None, peer_out_ptrs=None):
        assert peer_out_ptrs is None, "the CPU ranks must have agreed on the all-gather path"
        heads, sequence = prepared.sparse.heads, prepared.sparse.sequence
        head = torch.arange(self.first_head, self.first_head + heads, dtype=out.dtype).view(1, heads, 1, 1)
        row = torch.arange(sequence, dtype=out.dtype).view(1, 1, sequence, 1)
        out.copy_((head * 1000 + row).expand(1, heads, sequence, 128))
        return out


def _sharded_worker(rank, world, port, heads, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from h3_optimizations_b200.sharding import HeadShardedBackend

        a, b = head_partition(heads, world, rank)
        sharded = HeadShardedBackend(_StubBackend(a), heads, exchange="auto")
        sequence = 21
        q = torch.zeros((1, b - a, sequence, 128))
        prepared = sharded.prepare(q, q, q, layer_index=0, transformer_options={})
        full = sharded.execute(prepared)
        head = torch.arange(heads, dtype=torch.float32).view(1, heads, 1, 1)
        row = torch.arange(sequence, dtype=torch.float32).view(1, 1, sequence, 1)
        ok = torch.equal(full, (head * 1000 + row).expand(1, heads, sequence, 128))
        ok = ok and sharded.exchange == "nccl" and sharded.check_exchange(prepared)
        wrong = False
        try:
            sharded.prepare(torch.zeros((1, b - a + 1, sequence, 128)), q, q, layer_index=0, transformer_options={})
        except ValueError:
            wrong = True
        # the collective path is never recorded into a CUDA graph: capture refuses before it touches anything
        refused = False
        try:
            sharded.capture(q, q, q, layer_index=0, transformer_options={})
        except RuntimeError as exc:
            refused = "peer-store exchange" in str(exc)
        queue.put((rank, ok and wrong and refused))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("heads", [4, 5])
def test_head_sharded_backend_falls_back_to_the_collective_on_cpu_ranks(heads):
    """Without symmetric memory (CPU ranks here) every rank must agree on the
    all-gather path, and the reassembled output must be the full layer."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sharded_worker, args=(r, 2, port, heads, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
