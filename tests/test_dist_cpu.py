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


# ---------------------------------------------------------------------------------------------
# Tensor-parallel partition arithmetic on CPU ranks: every rank cuts its shard of a small model with
# weights.tp_shard_layer, runs the restated CPU forward over its shard with a gloo all-reduce where the
# engine all-reduces (after the out and down projections), and must reproduce the unsplit forward.
TP_DIMS = dict(hidden=64, n_layers=4, nq=4, nkv=2, head_dim=128, rot_dim=32, gdn_nk=2, gdn_nv=4, inter=128, vocab=50)


def _tp_worker(rank, world, port, out):
    from decide_b200.synth import synth_batch, synth_state_dict
    from decide_b200.weights import Dims, fuse_layer, tp_shard_layer
    from oracle import cpu_forward

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        d = Dims(**TP_DIMS)
        sd = synth_state_dict(d, seed=5)
        batch = synth_batch(d, 1, 21, seed=6, n_answers=2, n_cand=4, max_cand=4)
        positions = [int(r) for r in batch.ans_rows]
        cands = [batch.cand[i, :4] for i in range(2)]
        fused = [fuse_layer(sd, l, d) for l in range(d.n_layers)]
        local = [tp_shard_layer(fused[l], l, d, world, rank) for l in range(d.n_layers)]

        def all_reduce(a):
            t = torch.from_numpy(np.ascontiguousarray(a))
            dist.all_reduce(t)
            return t.numpy()

        got = cpu_forward.forward_logits(d.tp_local(world), local, sd["embed_tokens.weight"], sd["norm.weight"], batch.ids, positions, cands,
                                         all_reduce=all_reduce)
        want = cpu_forward.forward_logits(d, fused, sd["embed_tokens.weight"], sd["norm.weight"], batch.ids, positions, cands)
        out.put((rank, float(max(np.abs(g - w).max() for g, w in zip(got, want))), float(max(np.abs(w).max() for w in want))))
    finally:
        dist.destroy_process_group()


def test_tp_shards_reproduce_the_whole_model_on_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_tp_worker, args=(r, world, 29610, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, scale in results:
        assert err < 1e-4 * max(scale, 1.0), f"rank {rank}: sharded forward differs from the whole model by {err:.3e}"


def test_tp_local_dims_and_shapes():
    from decide_b200.synth import synth_state_dict
    from decide_b200.weights import BASELINE_DIMS, Dims, fuse_layer, tp_shard_layer

    for world in (2, 4, 8):
        loc = BASELINE_DIMS.tp_local(world)
        assert (loc.nq, loc.nkv, loc.gdn_nv, loc.inter) == (32 // world, 8 // world, 16 // world, 9728 // world)
        assert loc.lin_in_n % 32 == 0 and loc.att_in_n % 32 == 0 and loc.inter % 32 == 0 and loc.gate_cols == 16
    with pytest.raises(ValueError):
        BASELINE_DIMS.tp_local(3)
    d = Dims(**TP_DIMS)
    sd = synth_state_dict(d, seed=1)
    for l in (0, 3):
        whole = fuse_layer(sd, l, d)
        parts = [tp_shard_layer(whole, l, d, 2, r) for r in range(2)]
        loc = d.tp_local(2)
        assert all(p["w_in"].shape == ((loc.att_in_n if d.is_full_attention(l) else loc.lin_in_n), d.hidden) for p in parts)
        assert torch.equal(torch.cat([p["w_down"] for p in parts], dim=1), whole["w_down"])
        assert torch.equal(torch.cat([p["w_gu"] for p in parts], dim=0), whole["w_gu"])
        assert torch.equal(torch.cat([p["w_out"] for p in parts], dim=1), whole["w_out"])


@pytest.mark.parametrize("world", [4, 8])
def test_tp_shards_reproduce_the_whole_model_at_4_and_8_ranks(world):
    """The same partition arithmetic at the wider splits (one head of every kind per rank at 8), the ranks emulated as
    threads of one process whose all-reduce meets at a barrier: sums in rank order, so every rank sees the same bits."""
    import threading

    from decide_b200.synth import synth_batch, synth_state_dict
    from decide_b200.weights import Dims, fuse_layer, tp_shard_layer
    from oracle import cpu_forward

    d = Dims(hidden=64, n_layers=4, nq=8, nkv=8, head_dim=128, rot_dim=32, gdn_nk=8, gdn_nv=8, inter=256, vocab=50)
    sd = synth_state_dict(d, seed=7)
    batch = synth_batch(d, 1, 19, seed=8, n_answers=2, n_cand=4, max_cand=4)
    positions = [int(r) for r in batch.ans_rows]
    cands = [batch.cand[i, :4] for i in range(2)]
    fused = [fuse_layer(sd, l, d) for l in range(d.n_layers)]
    want = cpu_forward.forward_logits(d, fused, sd["embed_tokens.weight"], sd["norm.weight"], batch.ids, positions, cands)
    barrier, parts, got, errors = threading.Barrier(world), [None] * world, [None] * world, []

    def rank_main(rank):
        def all_reduce(a):
            parts[rank] = np.array(a, dtype=np.float64 if a.dtype == np.float64 else a.dtype)
            barrier.wait(timeout=120)
            total = parts[0].copy()
            for r in range(1, world):
                total = total + parts[r]
            barrier.wait(timeout=120)   # nobody overwrites its part before everybody has summed
            return total

        try:
            local = [tp_shard_layer(fused[l], l, d, world, rank) for l in range(d.n_layers)]
            got[rank] = cpu_forward.forward_logits(d.tp_local(world), local, sd["embed_tokens.weight"], sd["norm.weight"], batch.ids, positions, cands,
                                                   all_reduce=all_reduce)
        except Exception as e:   # a rank that fails must not leave the others at the barrier
            errors.append((rank, repr(e)))
            barrier.abort()

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    scale = max(np.abs(w).max() for w in want)
    for rank in range(world):
        err = max(np.abs(g - w).max() for g, w in zip(got[rank], want))
        assert err < 1e-4 * max(scale, 1.0), f"rank {rank} of {world}: sharded forward differs from the whole model by {err:.3e}"
        assert all(np.array_equal(a, b) for a, b in zip(got[rank], got[0]))
