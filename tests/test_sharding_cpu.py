"""N > 1 path on CPU: stream sharding and the max-over-ranks throughput reduction, world size 2, gloo."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from maskedincrementeval_b200.sharding import job_throughput, streams_of_rank
    mine = streams_of_rank(5, world, rank)
    steps = len(mine) * 10
    secs = 1.0 + rank          # rank 1 is the slow one
    dist.barrier()
    value, total, slowest = job_throughput(steps, secs)
    out.put((rank, mine, value, total, slowest))
    dist.destroy_process_group()


def test_streams_shard_round_robin():
    sys.path.insert(0, ROOT)
    from maskedincrementeval_b200.sharding import streams_of_rank
    assert streams_of_rank(8, 4, 1) == [1, 5]
    assert sorted(sum((streams_of_rank(7, 3, r) for r in range(3)), [])) == list(range(7))
    assert streams_of_rank(1, 8, 3) == []


def test_two_ranks_gloo_throughput_is_sum_over_slowest():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    (r0, s0, v0, t0, m0), (r1, s1, v1, t1, m1) = res
    assert s0 == [0, 2, 4] and s1 == [1, 3]
    assert t0 == t1 == 50 and m0 == m1 == 2.0
    assert abs(v0 - 25.0) < 1e-9 and abs(v1 - 25.0) < 1e-9
