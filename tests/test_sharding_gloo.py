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
