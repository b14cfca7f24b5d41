"""CPU, world size 2 over gloo: the host-side logic bench.py uses under torchrun — batch
sharding, the max-over-ranks reduction of the elapsed time and the verification gather."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    # strong scaling: contiguous batch shards that cover the batch exactly once
    lo, hi = bench.batch_shard(64, rank, world)
    spans = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(spans, torch.tensor([lo, hi]))
    # whole-job throughput uses the slowest rank
    ms = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    value = bench.job_throughput(tokens_per_rank=1000, world=world, steps=5, total_ms=float(ms))
    # verification gather of per-rank checksums
    chk = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(chk, torch.tensor([float(rank + 1)]))
    if rank == 0:
        out["spans"] = [s.tolist() for s in spans]
        out["ms"] = float(ms)
        out["value"] = value
        out["chk"] = [float(c) for c in chk]
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_gloo():
    mgr = mp.Manager()
    out = mgr.dict()
    port = 29600 + (os.getpid() % 200)
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    assert out["spans"] == [[0, 32], [32, 64]]
    assert out["ms"] == 11.0
    assert abs(out["value"] - 2 * 1000 * 5 / 11e-3) < 1e-6
    assert out["chk"] == [1.0, 2.0]


def test_batch_shard_edges():
    import bench
    assert bench.batch_shard(64, 0, 1) == (0, 64)
    cover = [bench.batch_shard(10, r, 4) for r in range(4)]
    assert cover[0][0] == 0 and cover[-1][1] == 10
    assert all(a[1] == b[0] for a, b in zip(cover, cover[1:]))
    assert max(h - l for l, h in cover) - min(h - l for l, h in cover) <= 1
