"""Parity table between this engine's candidate logits and gold logits: the rules of the reference's
`decide check` (crates/decide-cli/src/check.rs:22-25, 195-250).

Per answer row: max |dlogit|; max |dp| over the calibrated probabilities, which must stay within
MAX_DP = 0.01; the decision must agree wherever the gold's top-2 logit margin is at least
MARGIN = 0.05. A flip under that margin is a near-tie the tolerance cannot decide: it is reported as
a "small flip", not hidden and not failed, exactly as the reference does.
"""
from __future__ import annotations

import numpy as np

from . import head

MARGIN = 0.05
MAX_DP = 0.01
MAX_DLOGIT = 0.02  # the benchmark's bar on candidate logits


def top2_margin(logits: np.ndarray) -> float:
    """Difference of the two largest logits (head.rs top2_margin); inf for a single candidate."""
    x = np.sort(np.asarray(logits, dtype=np.float32))[::-1]
    return float(x[0] - x[1]) if len(x) > 1 else float("inf")


def compare(got: np.ndarray, want: np.ndarray, ncand) -> dict:
    """got, want: [n, max_cand] logits. Returns the parity table; `failures` is empty when every bar holds."""
    pg, dg = head.decide(got, ncand)
    pw, dw = head.decide(want, ncand)
    out = {"fields": len(ncand), "agree": 0, "max_dlogit": 0.0, "max_dp": 0.0, "small_flips": [], "failures": []}
    for i, n in enumerate(ncand):
        n = int(n)
        dl = float(np.abs(got[i, :n].astype(np.float64) - want[i, :n].astype(np.float64)).max())
        dp = float(np.abs(pg[i, :n] - pw[i, :n]).max())
        out["max_dlogit"] = max(out["max_dlogit"], dl)
        out["max_dp"] = max(out["max_dp"], dp)
        if not dl <= MAX_DLOGIT:
            out["failures"].append(f"row {i}: |dlogit| = {dl:.5f}, above {MAX_DLOGIT}")
        if not dp <= MAX_DP:
            out["failures"].append(f"row {i}: |dp| = {dp:.5f}, above {MAX_DP}")
        if dg[i] == dw[i]:
            out["agree"] += 1
        else:
            margin = top2_margin(want[i, :n])
            flip = f"row {i}: candidate {int(dg[i])}, gold {int(dw[i])} (gold top-2 margin {margin:.4f})"
            (out["failures"] if margin >= MARGIN else out["small_flips"]).append(("decision differs at " if margin >= MARGIN else "") + flip)
    return out
