"""Ties the two oracles together on the CPU: the Hugging Face model code that the reference's gold
generator runs (oracle/gold_synth.py, after reference/gold.py:32-63, 126-133) against the engine's
op sequence composed from the restated cpu_ref.rs functions over the FUSED weight layouts
(oracle/cpu_forward.py). Agreement pins (a) the restated kernels' semantics, (b) chunked (HF) vs
sequential (cpu_ref.rs) gated delta rule, (c) the converter layouts q|gate|k|v, qkv|z|b|a and the
gate|up interleave. Small dims so the pure-numpy side finishes in seconds."""
import numpy as np
import pytest

from decide_b200.synth import synth_batch, synth_state_dict
from decide_b200.weights import Dims, deinterleave_q_gate, fuse_layer, interleave_gate_up
from oracle import cpu_forward, gold_synth

SMALL = Dims(hidden=256, n_layers=4, nq=4, nkv=2, head_dim=128, rot_dim=128, gdn_nk=16, gdn_nv=16, inter=512, vocab=1000)
# the reference checkpoint's shape family: 2 value heads per key head, partial rotary
REFLIKE = Dims(hidden=256, n_layers=4, nq=4, nkv=1, head_dim=128, rot_dim=32, gdn_nk=8, gdn_nv=16, inter=256, vocab=500, rope_theta=1e7)


@pytest.mark.parametrize("dims,tokens", [(SMALL, 70), (REFLIKE, 33)], ids=["baseline-like", "reference-like"])
def test_hf_gold_equals_cpu_ref_composition(dims, tokens):
    sd = synth_state_dict(dims, seed=3)
    model = gold_synth.build_model(dims, sd)
    batch = synth_batch(dims, 1, tokens, seed=4, n_answers=3, n_cand=5, max_cand=8)
    want, _ = gold_synth.gold_batch_logits(model, batch, 8)
    fused = [fuse_layer(sd, l, dims) for l in range(dims.n_layers)]
    layers = []
    got = cpu_forward.forward_logits(dims, fused, sd["embed_tokens.weight"], sd["norm.weight"], batch.ids, batch.ans_rows,
                                     [batch.cand[i, :batch.ncand[i]] for i in range(len(batch.ans_rows))], layer_outputs=layers)
    hf_layers = gold_synth.gold_layer_outputs(model, batch.ids)
    for l, (a, b) in enumerate(zip(layers, hf_layers)):
        assert np.abs(a - b).max() < 2e-4 * max(1.0, np.abs(b).max()), f"residual after layer {l} differs"
    for i, g in enumerate(got):
        assert np.abs(g - want[i, :len(g)]).max() < 5e-4, f"answer {i}"


def test_fused_layout_helpers():
    import torch

    q = torch.arange(2 * 2 * 4 * 3, dtype=torch.float32).reshape(16, 3)  # 2 heads x (4 query + 4 gate rows)
    out = deinterleave_q_gate(q, heads=2, head_dim=4)
    assert torch.equal(out[:4], q[:4]) and torch.equal(out[4:8], q[8:12])      # queries of head 0, head 1
    assert torch.equal(out[8:12], q[4:8]) and torch.equal(out[12:], q[12:])    # gates of head 0, head 1
    gate = torch.arange(32, dtype=torch.float32).reshape(32, 1)
    up = gate + 100
    gu = interleave_gate_up(gate, up, 16)
    assert torch.equal(gu[:16], gate[:16]) and torch.equal(gu[16:32], up[:16]) and torch.equal(gu[32:48], gate[16:])


def test_synth_is_deterministic_and_layer_local():
    a = synth_state_dict(SMALL, seed=7)
    b = synth_state_dict(Dims(**{**SMALL.__dict__, "n_layers": 2}), seed=7)
    for k, v in b.items():
        assert (a[k] == v).all(), k
