"""Request JSON -> response JSON on the GPU (decide_b200/decision.py, the reference's Engine::decide,
crates/decide-engine/src/engine.rs:236-265) with synthetic weights and a byte-level tokenizer: the prompt stage, the
prefix snapshot, the state cache for follow-up questions, the prefill and the response builder in one call. The logits
are checked against the fp32 CPU gold forward on the same ids."""
import json

import numpy as np
import pytest

from decide_b200 import prompt
from decide_b200.decision import DecisionEngine
from decide_b200.synth import Batch
from oracle import gold_synth
from tests.test_model_gpu import SMALL, check_parity, make
from tests.test_prompt import byte_level_tokenizer_file

pytestmark = pytest.mark.gpu

STATE = {"ticket": "The customer was charged twice and asks for the extra payment back.", "amount": 12.5, "days_open": 3}
FIRST = {"team": {"type": "choice", "instructions": "Which team should handle this?", "criteria": {"billing": "Payments", "delivery": "Shipping", "other": "Else"}},
         "urgency": {"type": "score", "instructions": "Rate the priority.", "criteria": ["Low", "Medium", "High"]}}
SECOND = {"refund": {"type": "noul", "instructions": "Is the customer asking for a refund?"},
          "tone": {"type": "choice", "criteria": {"calm": "Neutral wording", "angry": "Hostile wording"}}}


def test_decide_cold_then_follow_up(dev, tmp_path):
    byte_level_tokenizer_file(tmp_path / "tokenizer.json")
    tok = prompt.Tokenizer.from_file(tmp_path / "tokenizer.json")
    sd, eng = make(SMALL, dev, 61, max_rows=2048, max_seqs=1, max_answers=16, max_cand=8)
    de = DecisionEngine(eng, tok)
    prefix = len(tok.prefix_ids())
    try:
        first = de.decide(json.dumps({"state": STATE, "questions": FIRST}))
        assert first.route == "snapshot" and first.rows == max(first.prepared.positions) + 1 - prefix
        boundary = eng.cached_states()
        assert len(boundary) == 1 and prefix < boundary[0] <= min(first.prepared.positions)
        follow = de.decide(json.dumps({"state": STATE, "questions": SECOND}))
        assert follow.route == "state_cache" and follow.rows == max(follow.prepared.positions) + 1 - boundary[0] < first.rows
        other = de.decide(json.dumps({"state": dict(STATE, days_open=4), "questions": SECOND}))     # another state: cold
        assert other.route == "snapshot" and len(eng.cached_states()) == 2
        # the follow-up's logits are those of a cold run of the same request
        eng.set_state_cache(0)
        cold = de.decide(json.dumps({"state": STATE, "questions": SECOND}))
        assert cold.route == "snapshot"
        for a, b in zip(follow.logits, cold.logits):
            assert np.abs(np.array(a) - np.array(b)).max() < 2e-3
        # the response: the reference's shape, one decision per field out of its options
        r = follow.response
        assert list(r) == ["answers", "usage", "timing", "calibration", "model", "backend"] and r["backend"] == "decide-cuda"
        assert r["usage"] == {"input_tokens": len(follow.prepared.ids), "output_tokens": 2, "decision_count": 2}
        assert list(r["answers"]) == ["refund", "tone"]
        assert r["answers"]["refund"]["decision"] in ("no", "yes") and r["answers"]["tone"]["choice"] in ("calm", "angry")
        assert abs(sum(r["answers"]["tone"]["probabilities"].values()) - 1.0) < 1e-9
        assert json.loads(follow.text()) == r
        assert first.response["answers"]["urgency"]["legend"] == {"0": "Low", "1": "Medium", "2": "High"}
        # against the fp32 CPU forward on the same ids
        p = first.prepared
        cand = np.zeros((2, 8), np.uint32)
        for i, c in enumerate(p.candidates):
            cand[i, :len(c)] = c
        batch = Batch(np.asarray(p.ids, np.uint32), np.array([0, len(p.ids)], np.uint32), np.asarray(p.positions, np.uint32), cand,
                      np.array([len(c) for c in p.candidates], np.uint32))
        want, _ = gold_synth.gold_batch_logits(gold_synth.build_model(SMALL, sd), batch, 8)
        got = np.zeros_like(want)
        for i, row in enumerate(first.logits):
            got[i, :len(row)] = row
        check_parity(got, want, batch.ncand, "decide (snapshot route)")
    finally:
        eng.build_snapshot([])
    eng.close()


def test_decide_check_against_gold_files_of_the_cpu_forward(dev, tmp_path):
    """`decide check` end to end (decide_b200/gold_check.py, crates/decide-cli/src/check.rs): gold files written from the
    fp32 CPU forward on the same synthetic weights (the layout reference/gold.py writes), then every request through the
    GPU engine: prompts and response envelopes identical, decisions and calibrated probabilities within the criteria."""
    from decide_b200 import gold_check, respond
    from decide_b200.decision import fields_of

    byte_level_tokenizer_file(tmp_path / "tokenizer.json")
    tok = prompt.Tokenizer.from_file(tmp_path / "tokenizer.json")
    sd, eng = make(SMALL, dev, 62, max_rows=2048, max_seqs=1, max_answers=16, max_cand=8)
    model = gold_synth.build_model(SMALL, sd)
    requests = {"core/first": {"state": STATE, "questions": FIRST}, "core/second": {"state": STATE, "questions": SECOND},
                "extra/other": {"state": {"note": "late parcel"}, "questions": SECOND}}
    for name, req in requests.items():
        text = json.dumps(req)
        p = tok.prepare(text)
        cand = np.zeros((len(p.positions), 8), np.uint32)
        for i, c in enumerate(p.candidates):
            cand[i, :len(c)] = c
        batch = Batch(np.asarray(p.ids, np.uint32), np.array([0, len(p.ids)], np.uint32), np.asarray(p.positions, np.uint32), cand,
                      np.array([len(c) for c in p.candidates], np.uint32))
        want, sec = gold_synth.gold_batch_logits(model, batch, 8)
        logits = [[float(x) for x in want[i, :len(c)]] for i, c in enumerate(p.candidates)]
        gold = {"name": name, "mode": "fp32", "input_ids": p.ids, "positions": p.positions, "fields": p.compiled.fields,
                "candidate_ids": dict(zip(p.compiled.fields, p.candidates)), "logits": dict(zip(p.compiled.fields, logits)),
                "response": respond.respond(fields_of(p), logits, len(p.ids), 1e3 * sec, backend="hf"), "seconds": sec}
        for root, obj in (("gold", gold), ("requests", req)):
            path = tmp_path / root / f"{name}.json"
            path.parent.mkdir(parents=True, exist_ok=True)
            path.write_text(json.dumps(obj))
    de = DecisionEngine(eng, tok)
    try:
        ok, lines = gold_check.check(de.decide, tmp_path / "gold", tmp_path / "requests")
    finally:
        eng.build_snapshot([])
    text = "\n".join(lines)
    print(text)
    assert ok, text
    assert "summary: 3 requests, 6 fields: PASS" in text and "prompts identical to the gold's (ids, logit rows, fields, candidates): 3/3" in text
    routes = [l.split()[2] for l in lines[4:7]]
    assert routes == ["snapshot", "state_cache", "snapshot"]
    eng.close()
