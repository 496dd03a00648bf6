"""BASELINE configs[2] and configs[3] at their stated size, M = 2,307 rows: ONE full-attention layer
(RMSNorm -> fused in-projection -> q/k head norm + RoPE -> causal GQA attention -> o-projection +
residual), gated (N = 10,240, the layout of the reference, forward.rs:105-107) and un-gated
(N = 6,144, the layout the benchmark description names), and ONE Gated DeltaNet layer (RMSNorm ->
in-projection N = 8,224 -> conv + SiLU + L2 -> chunk-64 gated delta rule over 37 chunks -> gated
RMSNorm -> out-projection + residual), at the benchmark's widths.

Each runs as a one-layer model through dc_model_prefill and is compared with the op sequence of
the reference's Forward over the restated cpu_ref.rs kernels (oracle/cpu_forward.py), rounding the
16-bit tensors where the engine rounds them: the residual stream after the layer over all 2,307
rows, and the candidate logits against the unrounded fp32 forward under the end-to-end bars. The
MLP that follows the mixer in a layer is kept narrow (it is not part of these configs)."""
import numpy as np
import pytest
import torch

from decide_b200.synth import synth_batch, synth_state_dict
from decide_b200.weights import BASELINE_DIMS, Dims, fuse_layer
from oracle import cpu_forward
from tests.test_model_gpu import check_parity

pytestmark = pytest.mark.gpu

T = 2307


def one_layer(kind: str) -> Dims:
    base = {**BASELINE_DIMS.__dict__, "n_layers": 1, "inter": 1024, "vocab": 4096}
    if kind == "gdn":
        return Dims(**{**base, "full_attn_interval": 4})        # layer 0 is a Gated DeltaNet layer
    return Dims(**{**base, "full_attn_interval": 1, "attn_gate": kind == "attention-gated"})


@pytest.mark.parametrize("kind", ["attention-gated", "attention-ungated", "gdn"])
def test_one_layer_at_2307_rows(dev, kind):
    from decide_b200.engine import Engine

    dims = one_layer(kind)
    sd = synth_state_dict(dims, seed=31)
    eng = Engine(dims, sd, dev=dev, max_rows=T, max_seqs=1, max_answers=4, max_cand=16)
    batch = synth_batch(dims, 1, T, seed=32, n_answers=3, n_cand=16, max_cand=16)
    eng.set_pruning(False)       # the residual of every row is wanted: no pruning, no truncation
    eng.set_truncation(False)
    got = eng.logits(batch)
    x_gpu = eng.buffer("x", (T, dims.hidden))
    eng.set_pruning(True)
    eng.set_truncation(True)
    skipping = eng.logits(batch)  # and the default, work-skipping pass gives the same logits
    eng.close()
    assert np.abs(skipping - got).max() < 2e-3

    fused = [fuse_layer(sd, 0, dims)]
    positions = [int(r) for r in batch.ans_rows]
    cands = [batch.cand[i, :batch.ncand[i]] for i in range(len(positions))]
    rounded_layers, exact_layers = [], []
    cpu_forward.forward_logits(dims, fused, sd["embed_tokens.weight"], sd["norm.weight"], batch.ids, positions, cands,
                               round_to="f16" if dev.act_torch == torch.float16 else "bf16", layer_outputs=rounded_layers)
    want = cpu_forward.forward_logits(dims, fused, sd["embed_tokens.weight"], sd["norm.weight"], batch.ids, positions, cands, layer_outputs=exact_layers)
    # the residual after the layer, all rows, against the CPU forward that rounds where the engine rounds
    x_cpu = rounded_layers[0]
    scale = np.abs(x_cpu).max()
    rel = np.abs(x_gpu - x_cpu).max() / scale
    rel_exact = np.abs(x_gpu - exact_layers[0]).max() / scale
    print(f"{kind} at {T} rows: residual differs by {rel:.2e} of its range from the rounding-matched CPU forward, {rel_exact:.2e} from fp32")
    assert np.isfinite(x_gpu).all()
    assert rel < 2e-3, f"{kind}: residual after the layer differs by {rel:.3e} of its range"
    # per-row: no single row is far off (a wrong chunk or tile would be a row-local error)
    row_err = np.abs(x_gpu - x_cpu).max(axis=1) / scale
    assert row_err.max() < 2e-3 and np.median(row_err) < 5e-4
    check_parity(got, np.stack([np.pad(np.asarray(l, np.float32), (0, 16 - len(l))) for l in want]), batch.ncand, f"{kind} logits")
