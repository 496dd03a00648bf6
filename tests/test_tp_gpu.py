"""Tensor-parallel prefill on 2 GPUs against the fp32 CPU gold forward and against the one-GPU engine.

One process per GPU (children of this test), each holding one rank's shard (heads and the MLP's
intermediate columns split, weights.tp_shard_layer); the partial sums of the out and down
projections are all-reduced over NCCL. The logits must meet the end-to-end bars against the gold
and sit within fp32-summation distance of the one-GPU engine's. Skipped on a single-GPU machine;
the partition arithmetic itself is also checked on CPU ranks (tests/test_dist_cpu.py).

The children only ever leave between steps; NVLS is off in them, and the parent kills by PID a child
that outlives its partner."""
import os

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from decide_b200.synth import synth_batch, synth_state_dict
from decide_b200.weights import BASELINE_DIMS, Dims

pytestmark = pytest.mark.gpu

SMALL_TP = Dims(hidden=256, n_layers=4, nq=4, nkv=2, head_dim=128, rot_dim=128, gdn_nk=16, gdn_nv=16, inter=512, vocab=1000)
WIDE_TP = Dims(**{**BASELINE_DIMS.__dict__, "n_layers": 4, "vocab": 4096})


def _rank(rank, world, uid, dims_kw, seed, batch_args, out):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        from decide_b200.engine import Engine
        from decide_b200.kernels import Device

        dims = Dims(**dims_kw)
        torch.cuda.set_device(rank)
        dev = Device(rank)
        dev.tp_init(uid, world, rank)
        sd = synth_state_dict(dims, seed)
        n_req, tokens, bseed = batch_args
        batch = synth_batch(dims, n_req, tokens, seed=bseed, n_answers=3, n_cand=8, max_cand=8)
        eng = Engine(dims, sd, dev=dev, max_rows=n_req * tokens, max_seqs=n_req, max_answers=3 * n_req, max_cand=8)
        first = eng.logits(batch)
        again = eng.logits(batch)
        dev.check_status()
        out.put((rank, first, bool(np.array_equal(first, again)), None))
        eng.close()
        dev.close()
    except Exception as e:  # the parent fails the test with this text
        out.put((rank, None, False, repr(e)))


def _run_tp(world, dims, seed, batch_args):
    from decide_b200.kernels import Device

    uid = Device.tp_unique_id()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, world, uid, dims.__dict__, seed, batch_args, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, logits, same, err = out.get(timeout=600)
            assert err is None, f"rank {rank}: {err}"
            results[rank] = (logits, same)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return results


@pytest.mark.parametrize("which", ["small", "benchmark-widths"])
def test_two_way_tensor_parallel_prefill(dev, which):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from decide_b200 import check
    from decide_b200.engine import Engine
    from oracle import gold_synth

    dims, batch_args = (SMALL_TP, (3, 90, 4)) if which == "small" else (WIDE_TP, (1, 603, 5))
    seed = 17
    results = _run_tp(2, dims, seed, batch_args)
    assert np.array_equal(results[0][0], results[1][0]), "the ranks of a group must hold identical logits"
    assert results[0][1] and results[1][1], "two passes over one batch differ"
    got = results[0][0]
    sd = synth_state_dict(dims, seed)
    n_req, tokens, bseed = batch_args
    batch = synth_batch(dims, n_req, tokens, seed=bseed, n_answers=3, n_cand=8, max_cand=8)
    want, _ = gold_synth.gold_batch_logits(gold_synth.build_model(dims, sd), batch, 8)
    t = check.compare(got, want, batch.ncand)
    assert not t["failures"], t["failures"]
    eng = Engine(dims, sd, dev=dev, max_rows=n_req * tokens, max_seqs=n_req, max_answers=3 * n_req, max_cand=8)
    one = eng.logits(batch)
    eng.close()
    d = float(np.abs(got - one).max())
    print(f"TP=2 {which}: max|dlogit| {t['max_dlogit']:.5f} vs gold, {d:.2e} vs the one-GPU engine")
    assert d < 5e-3
