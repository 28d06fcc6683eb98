"""The multi-rank plumbing of bench.py on CPU: two gloo ranks, each with its own timings; rank 0
must report the slowest rank's figures, and the aggregate of a replicated workload is world x
per-rank work / slowest time."""
import os
import sys

import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import bench
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    assert bench.dist_env() == (rank, world, rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = [1.0 + rank, 5.0 - rank, 2.5]
    got = bench.max_over_ranks(mine)
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, got))


def test_max_over_ranks_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29641, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0] == [2.0, 5.0, 2.5] and res[1] == [2.0, 5.0, 2.5]


def test_max_over_ranks_without_process_group():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.max_over_ranks([3.0, 1.0]) == [3.0, 1.0]
