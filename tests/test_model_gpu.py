"""Whole-model prefill on the GPU against the reference's fp32 CPU gold forward (the Hugging Face
model code reference/gold.py runs, oracle/gold_synth.py) on the same seeded random-init weights and
token ids. Bars (the reference's `decide check`, crates/decide-cli/src/check.rs:22-25, and the
benchmark's): max |dlogit| <= 0.02 on candidate logits, calibrated max |dp| <= 0.01, identical
argmax decisions. Per-layer residual comparison follows the reference's debug_layers
(forward.rs:778-797) against gold.py's hidden-state hooks (gold.py:115-118)."""
import numpy as np
import pytest

from decide_b200 import check
from decide_b200.synth import Batch, synth_batch, synth_state_dict
from decide_b200.weights import BASELINE_DIMS, Dims
from oracle import gold_synth

pytestmark = pytest.mark.gpu

SMALL = Dims(hidden=256, n_layers=4, nq=4, nkv=2, head_dim=128, rot_dim=128, gdn_nk=16, gdn_nv=16, inter=512, vocab=1000)
REFLIKE = Dims(hidden=256, n_layers=4, nq=4, nkv=1, head_dim=128, rot_dim=32, gdn_nk=8, gdn_nv=16, inter=256, vocab=500, rope_theta=1e7)

def check_parity(got, want, ncand, what):
    """max |dlogit| <= 0.02, calibrated max |dp| <= 0.01, decisions equal wherever the gold top-2 logit
    margin is >= 0.05 (check.rs:22-25); near-tie flips under that margin are printed, not failed."""
    t = check.compare(got, want, ncand)
    assert not t["failures"], f"{what}: {t['failures']}"
    if t["small_flips"]:
        print(f"{what}: near-tie flips (gold margin < {check.MARGIN}): {t['small_flips']}")
    return t["max_dlogit"], t["max_dp"]


def make(dims, dev, seed, **kw):
    from decide_b200.engine import Engine

    sd = synth_state_dict(dims, seed)
    return sd, Engine(dims, sd, dev=dev, **kw)


@pytest.mark.parametrize("dims", [SMALL, REFLIKE], ids=["baseline-like", "reference-like"])
def test_small_model_logits_and_layers(dev, dims, act):
    sd, eng = make(dims, dev, 3, max_rows=512, max_seqs=4, max_answers=16, max_cand=8)
    model = gold_synth.build_model(dims, sd)
    lens = [70, 9, 131]
    parts = [synth_batch(dims, 1, n, seed=10 + n, n_answers=3, n_cand=5, max_cand=8) for n in lens]
    starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    batch = Batch(np.concatenate([p.ids for p in parts]), starts,
                  np.concatenate([p.ans_rows + starts[i] for i, p in enumerate(parts)]).astype(np.uint32),
                  np.concatenate([p.cand for p in parts]), np.concatenate([p.ncand for p in parts]))
    want, _ = gold_synth.gold_batch_logits(model, batch, 8)
    got = eng.logits(batch)
    check_parity(got, want, batch.ncand, "small model")
    # residual stream after each layer, request 0
    hf_layers = gold_synth.gold_layer_outputs(model, parts[0].ids)
    for l in range(dims.n_layers):
        eng.set_layer_limit(l + 1)
        eng.logits(batch)
        x = eng.buffer("x", (batch.rows, dims.hidden))[:lens[0]]
        rel = np.abs(x - hf_layers[l]).max() / np.abs(hf_layers[l]).max()
        assert rel < 2e-2, f"layer {l}: residual differs by {rel:.3e} of its range"
    eng.set_layer_limit(0)
    eng.close()


def test_request_alone_equals_request_in_a_batch(dev):
    """Results must not depend on how requests are batched (the reference's chunk-size invariance,
    forward.rs:504-510, in this engine's terms) beyond fp32 summation order in the delta rule."""
    sd, eng = make(SMALL, dev, 5, max_rows=512, max_seqs=8, max_answers=64, max_cand=8)
    batch = synth_batch(SMALL, 4, 50, seed=6, n_answers=2, n_cand=8, max_cand=8)
    whole = eng.logits(batch)
    for s in range(4):
        one = Batch(batch.ids[s * 50:(s + 1) * 50].copy(), np.array([0, 50], np.uint32), batch.ans_rows[2 * s:2 * s + 2] - np.uint32(s * 50),
                    batch.cand[2 * s:2 * s + 2].copy(), batch.ncand[2 * s:2 * s + 2].copy())
        alone = eng.logits(one)
        assert np.abs(alone - whole[2 * s:2 * s + 2]).max() < 1e-4
    # the same batch twice is bit-identical
    assert np.array_equal(eng.logits(batch), whole)
    eng.close()


def test_engines_agree_on_the_whole_model(dev):
    """The same batch through the tcgen05 kernels (delta rule with the conv fused in, attention) and through
    the mma.sync kernels (separate conv): identical decisions, logits within a fraction of the gold tolerance."""
    from decide_b200.kernels import Engine as Eng, Family

    sd, eng = make(SMALL, dev, 21, max_rows=1024, max_seqs=4, max_answers=16, max_cand=8)
    batch = synth_batch(SMALL, 3, 200, seed=22, n_answers=3, n_cand=8, max_cand=8)
    try:
        tc = eng.logits(batch)
        for fam in (Family.Attn, Family.Delta):
            dev.set_engine(fam, Eng.MmaSync)
        legacy = eng.logits(batch)
    finally:
        for fam in (Family.Attn, Family.Delta):
            dev.set_engine(fam, Eng.Tcgen05)
    dev.check_status()
    assert np.abs(tc - legacy).max() < 2e-3, f"engines differ by {np.abs(tc - legacy).max():.2e}"
    assert np.isfinite(tc).all()
    eng.close()


def test_baseline_dims_four_layers(dev):
    """3 Gated DeltaNet layers + 1 attention layer at the benchmark's widths, two 603-token requests."""
    dims = Dims(**{**BASELINE_DIMS.__dict__, "n_layers": 4})
    sd, eng = make(dims, dev, 11, max_rows=1280, max_seqs=2, max_answers=12, max_cand=16)
    model = gold_synth.build_model(dims, sd)
    batch = synth_batch(dims, 2, 603, seed=12)
    want, _ = gold_synth.gold_batch_logits(model, batch, 16)
    got = eng.logits(batch)
    dl, dp = check_parity(got, want, batch.ncand, "4 layers at benchmark widths")
    hf_layers = gold_synth.gold_layer_outputs(model, batch.ids[:603])
    for l in range(4):
        eng.set_layer_limit(l + 1)
        eng.logits(batch)
        x = eng.buffer("x", (batch.rows, dims.hidden))[:603]
        rel = np.abs(x - hf_layers[l]).max() / np.abs(hf_layers[l]).max()
        assert rel < 1e-2, f"layer {l}: residual differs by {rel:.3e} of its range"
    eng.set_layer_limit(0)
    eng.close()


def test_full_model_parity(dev):
    """BASELINE config 4 in small: the full 36-layer model, 603-token requests, 6 answer rows x 16
    candidates each, against the fp32 CPU gold forward."""
    dims = BASELINE_DIMS
    sd, eng = make(dims, dev, 1, max_rows=2 * 603, max_seqs=2, max_answers=12, max_cand=16)
    model = gold_synth.build_model(dims, sd)
    batch = synth_batch(dims, 2, 603, seed=2)
    want, secs = gold_synth.gold_batch_logits(model, batch, 16)
    got = eng.logits(batch)
    dl, dp = check_parity(got, want, batch.ncand, "full model")
    print(f"full model: max|dlogit| {dl:.5f} max|dp| {dp:.5f}; CPU gold {secs:.1f}s for 2 requests")
    eng.close()


def test_prefill_argument_checks(dev):
    from decide_b200.kernels import KernelError

    sd, eng = make(SMALL, dev, 5, max_rows=64, max_seqs=2, max_answers=4, max_cand=8)
    ok = synth_batch(SMALL, 1, 20, seed=1, n_answers=2, n_cand=4, max_cand=8)
    eng.logits(ok)
    bad_rows = synth_batch(SMALL, 1, 100, seed=1, n_answers=2, n_cand=4, max_cand=8)
    with pytest.raises(KernelError):
        eng.logits(bad_rows)
    bad_id = Batch(ok.ids.copy(), ok.seq_start, ok.ans_rows, ok.cand, ok.ncand)
    bad_id.ids[3] = SMALL.vocab
    with pytest.raises(KernelError):
        eng.logits(bad_id)
    bad_ans = Batch(ok.ids, ok.seq_start, np.array([5, 20], np.uint32), ok.cand, ok.ncand)
    with pytest.raises(KernelError):
        eng.logits(bad_ans)
    eng.logits(ok)  # still usable after refused calls
    eng.close()
