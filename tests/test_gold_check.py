"""`decide check` host logic (decide_b200/gold_check.py, crates/decide-cli/src/check.rs) on the reference's 58 gold
responses: a stand-in engine that answers with the gold's own logits must PASS with every prompt and envelope equal;
a shifted logit, a reordered response and a changed prompt must each FAIL with the reference's kind of message."""
import copy
import json
from pathlib import Path
from types import SimpleNamespace

import pytest

from decide_b200 import gold_check, respond
from decide_b200.decision import Decision

GOLDEN = Path(__file__).parent / "golden"
RESP = {c["file"]: c for c in json.loads((GOLDEN / "response_kat.json").read_text())["cases"]}
REQ = {c["file"]: c for c in json.loads((GOLDEN / "request_kat.json").read_text())["cases"]}


def gold_of(file: str) -> dict:
    r, q = RESP[file], REQ[file]
    return {"input_ids": list(range(q["n_ids"])), "positions": q["positions"], "fields": q["fields"],
            "candidate_ids": dict(zip(q["fields"], q["candidate_ids"])), "logits": dict(zip(q["fields"], r["logits"])), "response": r["response"]}


def decision_of(file: str, shift: float = 0.0, route: str = "snapshot") -> Decision:
    r, q = RESP[file], REQ[file]
    fields = [respond.Field(f["name"], f["kind"], [tuple(o) for o in f["options"]]) for f in r["fields"]]
    logits = [[x + (shift if i == 0 else 0.0) for i, x in enumerate(row)] for row in r["logits"]]
    prepared = SimpleNamespace(ids=list(range(q["n_ids"])), positions=q["positions"], candidates=q["candidate_ids"],
                               compiled=SimpleNamespace(fields=q["fields"]))
    return Decision(respond.respond(fields, logits, q["n_ids"], 12.0), prepared, logits, route, 100, {"forward_ms": 12.0})


@pytest.fixture
def dirs(tmp_path):
    for file in RESP:
        for root, obj in (("gold", gold_of(file)), ("requests", {"file": file})):
            p = tmp_path / root / file
            p.parent.mkdir(parents=True, exist_ok=True)
            p.write_text(json.dumps(obj))
    return tmp_path / "gold", tmp_path / "requests"


def test_the_gold_against_itself_passes(dirs):
    ok, lines = gold_check.check(lambda text: decision_of(json.loads(text)["file"]), *dirs)
    text = "\n".join(lines)
    assert ok, text
    assert "summary: 58 requests" in text and "PASS" in text
    assert "prompts identical to the gold's (ids, logit rows, fields, candidates): 58/58" in text
    assert "aside): 58/58" in text and "from the prefix snapshot (or a cached state) 58/58" in text
    names = [l.split()[0] for l in lines[4:62]]
    assert names[0].startswith("core/") and names == sorted(names, key=lambda n: (not n.startswith("core/"), n))   # core first


def test_failures_are_named(dirs):
    def decide(text):
        file = json.loads(text)["file"]
        if file == "core/card.json":
            return decision_of(file, shift=1.0)              # probabilities move by more than 0.01
        d = decision_of(file, route="full")
        if file == "core/ticket6.json":
            d.response = {k: d.response[k] for k in reversed(list(d.response))}
        if file == "calib/calib_00.json":
            d.prepared.positions = [p + 1 for p in d.prepared.positions]
        if file == "calib/calib_01.json":
            raise ValueError("Supply 1–16 questions.")
        return d

    ok, lines = gold_check.check(decide, *dirs)
    text = "\n".join(lines)
    assert not ok and "FAIL" in text
    assert "core/card:" in text and "|dp| =" in text
    assert "response differs: core/ticket6: keys" in text
    assert "calib/calib_00: the prompt (ids, logit rows, fields or candidates) differs from the gold's" in text
    assert "calib/calib_01: the engine refused or failed the request: Supply 1–16 questions." in text
    assert "prompts identical to the gold's (ids, logit rows, fields, candidates): 56/58" in text


def test_same_shape_rules():
    out = []
    gold = {"a": {"type": "choice", "n": 3, "p": 0.25, "decision": "x", "flag": True}, "l": [1, "s"]}
    ours = copy.deepcopy(gold)
    ours["a"]["p"], ours["a"]["decision"] = 0.75, "y"        # floats and decisions are compared elsewhere
    gold_check.same_shape(ours, gold, "r", out)
    assert out == []
    ours["a"]["n"], ours["l"][1], ours["a"]["flag"] = 4, "t", 1
    gold_check.same_shape(ours, gold, "r", out)
    assert out == ["r.a.n: 4, gold 3", "r.a.flag: 1, gold true", 'r.l[1]: "t", gold "s"']
