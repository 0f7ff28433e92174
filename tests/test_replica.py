"""CPU: the multi-rank plumbing of the benchmark (sequence partition, counter reduction) with two gloo ranks."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    entry.load_package()
    import importlib
    replica = importlib.import_module(entry.PKG_NAME + ".replica")
    replica.init("gloo")
    mine = list(replica.partition(13, world, rank))
    ms = 100.0 + 50.0 * rank                   # rank 1 is the slow one
    tokens = float(len(mine) * 1536)
    mx, sm = replica.reduce_counters([ms], [tokens])
    replica.barrier()
    q.put((rank, mine, mx[0], sm[0], replica.job_throughput(sm[0], mx[0])))
    dist.destroy_process_group()


def test_two_ranks_partition_and_reduce():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    ps = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in ps]
    res = sorted(q.get(timeout=120) for _ in range(2))
    [p.join(timeout=60) for p in ps]
    assert all(p.exitcode == 0 for p in ps)
    (r0, s0, mx0, sm0, v0), (r1, s1, mx1, sm1, v1) = res
    assert sorted(s0 + s1) == list(range(13)) and not set(s0) & set(s1)       # every sequence on exactly one rank
    assert s0 == list(range(0, 13, 2)) and s1 == list(range(1, 13, 2))
    assert mx0 == mx1 == 150.0                                                 # max over ranks
    assert sm0 == sm1 == 13 * 1536.0                                           # units of all ranks
    assert abs(v0 - 13 * 1536 / 0.150) < 1e-6 and v0 == v1


def test_single_process_passthrough():
    entry.load_package()
    import importlib
    replica = importlib.import_module(entry.PKG_NAME + ".replica")
    assert replica.reduce_counters([3.0], [5.0]) == ([3.0], [5.0])
    assert list(replica.partition(5, 1, 0)) == [0, 1, 2, 3, 4]
