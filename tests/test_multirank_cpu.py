"""The N>1 path of the benchmark on CPU: two gloo ranks shard the batch with no data-path
collective; the only exchange is the MAX reduction of the per-rank elapsed time."""

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
    import bench
    from oracle import inputs
    # every rank draws its own shard (seed offset by rank): shards differ, shapes agree
    q, _, _ = inputs.attention_bshd(1, 2, 64, 64, 64, bench.C2["seed"] + rank)
    t = torch.tensor([10.0 + rank, 20.0 - rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out.put((rank, float(q.float().sum()), t.tolist(), bench.c2_flops() * world))
    dist.destroy_process_group()


def test_two_ranks_shard_and_reduce_max():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29611, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][1] != res[1][1]                       # different shards
    assert res[0][2] == res[1][2] == [11.0, 20.0]       # max over ranks on every rank
    assert res[0][3] == 2 * __import__("bench").c2_flops()
