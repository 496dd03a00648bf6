"""The post-logit head (softmax f32 -> temperature scaling f64 -> decision) against the reference's
own golden vectors: tests/golden/head_kat.json holds, for all 65 fields of the 58 gold fixtures, the
gold logits and the probabilities / decision the reference pipeline derived from them."""
import json
from pathlib import Path

import numpy as np
import pytest

from decide_b200 import head
from oracle import head_math

KAT = json.loads((Path(__file__).parent / "golden" / "head_kat.json").read_text())["cases"]


def test_kat_is_complete():
    assert len(KAT) == 65 and len({c["file"] for c in KAT}) == 58


@pytest.mark.parametrize("case", KAT, ids=lambda c: f"{c['file']}:{c['field']}")
def test_oracle_reproduces_reference_probabilities(case):
    assert case["temperature"] == head_math.TEMPERATURE
    p, best = head_math.calibrated(case["logits"], case["labels"], case["temperature"])
    # torch's softmax may differ from libm's by an ulp or two of f32 (head.rs:42-44)
    assert np.allclose(p, case["probabilities"], rtol=5e-6, atol=1e-9)
    assert case["labels"][best] == case["decision"]


def test_product_head_matches_oracle_on_every_kat_row():
    for case in KAT:
        probs, dec = head.decide(np.array([case["logits"]], dtype=np.float32))
        want, _ = head_math.calibrated(case["logits"], case["labels"], case["temperature"])
        assert np.allclose(probs[0], want, rtol=1e-6, atol=1e-12)
        assert case["labels"][dec[0]] == case["decision"]


def test_argmax_ties_go_to_the_smaller_label():
    assert head_math.argmax(["b", "a"], [0.5, 0.5]) == 1
    assert head_math.argmax(["a", "b"], [0.5, 0.5]) == 0
    assert head_math.argmax(["a", "b", "c"], [0.2, 0.5, 0.3]) == 1


def test_py_sum_is_compensated():
    assert head_math.py_sum([1e100, 1.0, -1e100]) == 1.0
    assert head_math.py_sum([]) == 0.0


def test_scale_probabilities_errors():
    with pytest.raises(ValueError):
        head_math.scale_probabilities(["a"], [1.0], 0.0)
    with pytest.raises(ValueError):
        head_math.scale_probabilities(["a", "b"], [0.7, 0.7], 2.0)
    with pytest.raises(ValueError):
        head.scale_probabilities(np.array([0.7, 0.7]), 2.0)
    assert head_math.scale_probabilities(["a", "b"], [0.25, 0.75], 1.0) == [0.25, 0.75]
    p = head_math.scale_probabilities(["a", "b"], [0.0, 1.0], 2.0)
    assert p == [0.0, 1.0]


def test_check_table_rules():
    """The parity table: |dlogit| and |dp| bars, and the margin rule for decisions (check.rs:22-25)."""
    from decide_b200 import check

    want = np.array([[2.0, 1.0, 0.0], [1.00, 0.99, 0.0], [1.0, 0.9, 0.0]], dtype=np.float32)
    got = want.copy()
    got[1] = [0.99, 1.0, 0.0]      # near-tie flip: gold margin 0.01 < 0.05
    t = check.compare(got, want, [3, 3, 3])
    assert t["failures"] == [] and len(t["small_flips"]) == 1 and t["agree"] == 2
    got[2] = [0.94, 0.96, 0.0]     # flip with gold margin 0.1 >= 0.05, and |dlogit| 0.06 > 0.02
    t = check.compare(got, want, [3, 3, 3])
    assert any("decision differs" in f for f in t["failures"]) and any("dlogit" in f for f in t["failures"])
    assert check.top2_margin(np.array([3.0])) == float("inf")
