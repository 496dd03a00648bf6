"""The response builder (decide_b200/respond.py) against the reference's own golden responses: for each
of its 58 gold fixtures, the response object its Python pipeline produced from the fp32 gold logits
(tests/golden/response_kat.json, extracted by tests/golden/make_response_kat.py)."""
import json
from pathlib import Path

import pytest

from decide_b200 import respond as R

KAT = json.loads((Path(__file__).parent / "golden" / "response_kat.json").read_text())["cases"]


def _fields(case):
    return [R.Field(f["name"], f["kind"], [tuple(o) for o in f["options"]]) for f in case["fields"]]


def _same(got, want, rel):
    """Same structure, keys in the same order, same strings and ints; floats within `rel`."""
    if isinstance(want, dict):
        assert isinstance(got, dict) and list(got) == list(want)
        for k in want:
            _same(got[k], want[k], rel)
    elif isinstance(want, float):
        assert isinstance(got, float) and abs(got - want) <= rel * max(abs(want), 1e-30), (got, want)
    else:
        assert got == want and type(got) is type(want)


def test_all_58_gold_responses():
    """The gold responses were made with torch.softmax, whose f32 values differ from the reference engine's own
    softmax formula (max, exp, sum, divide) by an ulp or two (head.rs:43-45 says so); everything downstream is exact.
    So: with this module's softmax (the engine's formula) every response matches in structure, key order, labels,
    decisions and integers, and in every float to a few f32 ulps; with torch's softmax injected, the JSON text itself
    is reproduced byte for byte (for all but the odd case where the installed torch rounds one exp differently)."""
    import torch

    assert len(KAT) == 58
    kinds, exact = set(), 0
    for case in KAT:
        got = R.respond(_fields(case), case["logits"], case["input_tokens"], case["inference_ms"], backend="hf")
        _same(got, case["response"], rel=3e-7)
        for name, ans in case["response"]["answers"].items():
            assert got["answers"][name]["decision"] == ans["decision"]
        kinds |= {f["kind"] for f in case["fields"]}
    assert kinds == {"choice", "score", "noul"}
    engine_softmax = R.softmax
    R.softmax = lambda row: torch.softmax(torch.tensor(row, dtype=torch.float32), dim=-1).tolist()
    try:
        for case in KAT:
            got = R.respond(_fields(case), case["logits"], case["input_tokens"], case["inference_ms"], backend="hf")
            exact += json.dumps(got) == json.dumps(case["response"])
    finally:
        R.softmax = engine_softmax
    assert exact >= 50, f"only {exact} of 58 gold responses reproduced byte for byte with torch's softmax"


def test_backend_name_and_rounded_time():
    case = KAT[0]
    got = R.respond(_fields(case), case["logits"], case["input_tokens"], 12.3456)
    assert got["backend"] == "decide-cuda" and got["timing"] == {"inference_ms": 12.35} and got["model"] == "Intern-Decision-4B"
    assert got["usage"] == {"input_tokens": case["input_tokens"], "output_tokens": len(case["fields"]), "decision_count": len(case["fields"])}


def test_refusals_of_the_reference():
    f = [R.Field("q", "choice", [("a", ""), ("b", "")])]
    with pytest.raises(R.HeadError, match="logit rows"):
        R.respond(f, [], 1, 1.0)
    with pytest.raises(R.HeadError, match="logits for the 2 options"):
        R.respond(f, [[0.0]], 1, 1.0)
    with pytest.raises(R.HeadError, match="Invalid probability"):
        R.respond(f, [[float("nan"), 0.0]], 1, 1.0)
    with pytest.raises(R.HeadError, match='no "yes" option'):
        R.respond([R.Field("q", "noul", [("no", ""), ("maybe", "")])], [[0.0, 1.0]], 1, 1.0)
    with pytest.raises(R.HeadError, match="could not convert"):
        R.respond([R.Field("q", "score", [("low", ""), ("1", "")])], [[0.0, 1.0]], 1, 1.0)
    # ties go to the smaller label, whatever the option order
    tie = R.respond([R.Field("q", "choice", [("b", ""), ("a", "")])], [[1.0, 1.0]], 1, 1.0)
    assert tie["answers"]["q"]["decision"] == "a"
