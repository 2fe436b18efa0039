"""CPU, world_size 2 over gloo: the replica plumbing bench.py uses at N > 1 -- shard ownership, the
max-over-ranks clock, the aggregate throughput and the check that every replica produced the same
logits for the same batch."""
import os
import socket

import pytest
import torch.multiprocessing as mp

from nart_b200 import replicas


def test_shard_partitions_the_batch():
    for total in (0, 1, 7, 256, 1000):
        for world in (1, 2, 3, 8):
            spans = [replicas.shard(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        replicas.shard(10, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    r, w = replicas.init("gloo")
    assert (r, w) == (rank, world)
    replicas.barrier()
    elapsed_ms = 100.0 * (rank + 1)            # rank 1 is the slow one
    slowest = replicas.max_over_ranks(elapsed_ms)
    ips = replicas.images_per_sec(256, 10, elapsed_ms)
    same = replicas.all_ranks_hold(b"digest-of-the-logits")
    differ = replicas.all_ranks_hold(b"rank %d" % rank)
    out.put((rank, slowest, ips, same, differ))
    import torch.distributed as dist
    dist.destroy_process_group()


def test_two_ranks_agree_on_the_slowest_clock_and_the_aggregate():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, slowest, ips, same, differ in got:
        assert slowest == 200.0
        assert abs(ips - 2 * 256 * 10 / 0.2) < 1e-6
        assert same is True and differ is False      # every rank learns whether the replicas agree
