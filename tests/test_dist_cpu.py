"""The multi-rank host logic on CPU ranks (gloo, world size 2 and 3): request sharding, the
max-over-ranks timing reduction and the gather of per-request logits on rank 0. No GPU involved:
the data path itself has no collective."""
import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from decide_b200 import dist as ddist


def test_shard_is_a_partition():
    for n in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 8):
            got = [i for r in range(world) for i in ddist.shard(n, world, r)]
            assert got == list(range(n))
            sizes = [len(ddist.shard(n, world, r)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        ddist.shard(4, 2, 2)


def test_single_process_is_identity():
    assert ddist.max_over_ranks(3.5) == 3.5
    x = np.arange(6, dtype=np.float32).reshape(3, 2)
    assert ddist.gather_rows(x) is x


def _worker(rank, world, port, out):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        n_req = 7
        mine = ddist.shard(n_req, world, rank)
        local = np.stack([np.full(4, 10.0 * i, dtype=np.float32) for i in mine]) if len(mine) else np.zeros((0, 4), np.float32)
        slowest = ddist.max_over_ranks(1.0 + rank)
        allrows = ddist.gather_rows(local)
        out.put((rank, slowest, None if allrows is None else allrows.tolist()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_gloo_ranks(world):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29600 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, slowest, rows = out.get(timeout=120)
        results[rank] = (slowest, rows)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(v[0] == float(world) for v in results.values())          # the slowest rank's time everywhere
    assert results[0][1] == [[10.0 * i] * 4 for i in range(7)]           # rank order = request order
    assert all(results[r][1] is None for r in range(1, world))
