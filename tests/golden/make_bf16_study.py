"""Generates tests/golden/bf16_study.json: what the 16-bit storage type of the activations costs in
candidate-logit error over the full 36-layer model, computed entirely on the CPU.

    python tests/golden/make_bf16_study.py [--tokens 160] [--seed 1]

The engine stores every GEMM input (normed rows, mixer outputs, the MLP intermediate) and the
attention q/k/v in one 16-bit type. This script runs oracle/cpu_forward.py (the restated
cpu_ref.rs kernels in the reference's op order) on seeded synthetic weights at the benchmark's
dims with those tensors rounded the way the engine rounds them, and compares each variant's
candidate logits with the unrounded fp32 forward:

  fp32            no rounding (the gold; also compared with the Hugging Face model code)
  f16             every 16-bit tensor rounded to fp16 (the engine's default, the reference's choice)
  bf16            every 16-bit tensor rounded to bf16 (the type the benchmark description names)
  bf16+exact(...) bf16, but the named projections read their input unrounded: what feeding those
                  GEMMs the activation as a hi + lo pair of bf16 values would achieve, at twice
                  their tensor-core work

The GPU test tests/test_model_gpu.py::test_bf16_engine_matches_its_cpu_emulation then checks that
the engine in bf16 mode reproduces the "bf16" row's logits, i.e. that the error is the format's and
not a kernel's. The vocabulary is cut to 4096 rows (only gathered rows are ever read).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from decide_b200 import check  # noqa: E402
from decide_b200.synth import synth_batch, synth_state_dict  # noqa: E402
from decide_b200.weights import BASELINE_DIMS, Dims, fuse_layer  # noqa: E402
from oracle import cpu_forward, gold_synth  # noqa: E402

STUDY_VOCAB = 4096
N_ANSWERS, N_CAND = 6, 16


def study_dims() -> Dims:
    return Dims(**{**BASELINE_DIMS.__dict__, "vocab": STUDY_VOCAB})


def study_batch(dims: Dims, tokens: int, seed: int):
    return synth_batch(dims, 1, tokens, seed=seed + 1, n_answers=N_ANSWERS, n_cand=N_CAND, max_cand=N_CAND)


def logits_of(dims, fused, sd, batch, **kw) -> np.ndarray:
    positions = [int(r) for r in batch.ans_rows]
    cands = [batch.cand[i, :batch.ncand[i]] for i in range(len(positions))]
    out = cpu_forward.forward_logits(dims, fused, sd["embed_tokens.weight"], sd["norm.weight"], batch.ids, positions, cands, **kw)
    return np.stack([np.asarray(l, dtype=np.float32) for l in out])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=160)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--out", default=str(Path(__file__).with_name("bf16_study.json")))
    args = ap.parse_args()

    dims = study_dims()
    sd = synth_state_dict(dims, args.seed)
    fused = [fuse_layer(sd, l, dims) for l in range(dims.n_layers)]
    batch = study_batch(dims, args.tokens, args.seed)

    variants = [
        ("fp32", dict()),
        ("f16", dict(round_to="f16")),
        ("bf16", dict(round_to="bf16")),
        ("bf16+exact(out,down)", dict(round_to="bf16", exact_inputs=("out", "down"))),
        ("bf16+exact(in,out,gate_up,down)", dict(round_to="bf16", exact_inputs=("in", "out", "gate_up", "down"))),
    ]
    logits, secs = {}, {}
    for name, kw in variants:
        t0 = time.perf_counter()
        logits[name] = logits_of(dims, fused, sd, batch, **kw)
        secs[name] = time.perf_counter() - t0
        print(f"{name}: {secs[name]:.1f} s", flush=True)
    gold, _ = gold_synth.gold_batch_logits(gold_synth.build_model(dims, sd), batch, N_CAND)

    rows = {}
    for name, _ in variants:
        t = check.compare(logits[name], logits["fp32"], batch.ncand)
        rows[name] = {"max_abs_dlogit_vs_fp32": t["max_dlogit"], "max_abs_dp_vs_fp32": t["max_dp"],
                      "decisions_agree": f"{t['agree']}/{t['fields']}", "meets_bars": not t["failures"]}
    hf = check.compare(logits["fp32"], gold, batch.ncand)
    # share of the projection FLOPs whose input would be fed as hi + lo (their tensor-core work doubles)
    per_row = {"in": 0.0, "out": 0.0, "gate_up": 0.0, "down": 0.0}
    for l in range(dims.n_layers):
        if dims.is_full_attention(l):
            per_row["in"] += 2.0 * dims.hidden * dims.att_in_n
            per_row["out"] += 2.0 * dims.q_dim * dims.hidden
        else:
            per_row["in"] += 2.0 * dims.hidden * dims.lin_in_n
            per_row["out"] += 2.0 * dims.value_dim * dims.hidden
        per_row["gate_up"] += 2.0 * dims.hidden * 2 * dims.inter
        per_row["down"] += 2.0 * dims.inter * dims.hidden
    total = sum(per_row.values())
    out = {
        "what": "candidate-logit error of the full 36-layer model on the CPU by 16-bit storage type of the activations",
        "made_by": "tests/golden/make_bf16_study.py", "seed": args.seed, "tokens": args.tokens, "vocab": STUDY_VOCAB,
        "answers": N_ANSWERS, "candidates": N_CAND, "bars": {"max_abs_dlogit": check.MAX_DLOGIT, "max_abs_dp": check.MAX_DP},
        "variants": rows,
        "fp32_restated_vs_hf_model": {"max_abs_dlogit": hf["max_dlogit"], "max_abs_dp": hf["max_dp"]},
        "extra_gemm_work_of_exact_inputs": {"out,down": (per_row["out"] + per_row["down"]) / total, "all": 1.0},
        "logits_bf16": [[float(v) for v in r] for r in logits["bf16"]],
        "logits_f16": [[float(v) for v in r] for r in logits["f16"]],
        "logits_fp32": [[float(v) for v in r] for r in logits["fp32"]],
    }
    Path(args.out).write_text(json.dumps(out, indent=1) + "\n")
    print(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
