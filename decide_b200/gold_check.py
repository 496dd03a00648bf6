"""`decide check`: every gold request through the engine, end to end (request JSON in, response out), against the fp32
gold files (crates/decide-cli/src/check.rs). Criteria as there: identical decisions wherever the gold's top-2 logit
margin is at least MARGIN, calibrated probabilities within MAX_DP; each request's prompt (ids, logit rows, fields,
candidate ids) must be the gold's exactly and its response must have the gold's keys in the gold's order, the same
strings and ints and the gold's `calibration` (`backend`, `timing` and other floats aside).

A gold directory holds `<set>/<name>.json` with `input_ids`, `positions`, `fields`, `candidate_ids`, `logits`,
`response` (what reference/gold.py writes); the requests directory holds `<set>/<name>.json` beside it.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

from .check import MARGIN, MAX_DP, top2_margin

SKIPPED_KEYS = ("decision", "choice", "backend", "timing")


def cases(gold: Path, requests: Path) -> list:
    """(name, gold path, request path): the `core` set first, then the others, each by file name (check.rs:39-63)."""
    sets = sorted((p.name for p in Path(gold).iterdir() if p.is_dir()), key=lambda s: (s != "core", s))
    out = []
    for s in sets:
        for path in sorted((Path(gold) / s).glob("*.json")):
            out.append((f"{s}/{path.stem}", path, Path(requests) / s / path.name))
    if not out:
        raise ValueError(f"no gold files in {gold}/<set>/")
    return out


def same_prompt(decision, gold: dict) -> bool:
    """Whether the prompt is the gold's: ids, logit rows, fields, candidates (check.rs:122-132)."""
    p = decision.prepared
    fields = list(gold["fields"])
    return (list(p.ids) == list(gold["input_ids"]) and list(p.positions) == list(gold["positions"]) and p.compiled.fields == fields
            and len(p.candidates) == len(fields) and all(list(c) == list(gold["candidate_ids"][f]) for f, c in zip(fields, p.candidates)))


def same_shape(ours, gold, path: str, out: list):
    """Same keys in the same order, equal strings, ints and bools at every level; floats and SKIPPED_KEYS are the caller's
    (check.rs:134-166)."""
    if isinstance(ours, dict) and isinstance(gold, dict):
        if list(ours) != list(gold):
            out.append(f"{path}: keys {list(ours)}, gold {list(gold)}")
            return
        for key, value in ours.items():
            if key not in SKIPPED_KEYS:
                same_shape(value, gold[key], f"{path}.{key}", out)
    elif isinstance(ours, list) and isinstance(gold, list) and len(ours) == len(gold):
        for i, (x, y) in enumerate(zip(ours, gold)):
            same_shape(x, y, f"{path}[{i}]", out)
    elif isinstance(ours, float) and isinstance(gold, float) and not isinstance(ours, bool):
        pass
    elif type(ours) is not type(gold) or ours != gold:
        out.append(f"{path}: {json.dumps(ours)}, gold {json.dumps(gold)}")


def _worst(a: float, b: float) -> float:
    return math.nan if math.isnan(a) or math.isnan(b) else max(a, b)


def compare(name: str, decision, gold: dict, tally: dict) -> dict:
    """One request against its gold: its row of the table; failures and totals go to `tally` (check.rs:168-260)."""
    import numpy as np

    fields = list(gold["fields"])
    if same_prompt(decision, gold):
        tally["prompts_equal"] += 1
    else:
        tally["failures"].append(f"{name}: the prompt (ids, logit rows, fields or candidates) differs from the gold's")
    shape = []
    same_shape(decision.response, gold["response"], name, shape)
    if decision.response.get("calibration") != gold["response"].get("calibration"):
        shape.append(f"{name}.calibration: {decision.response.get('calibration')}, gold {gold['response'].get('calibration')}")
    if shape:
        tally["failures"] += [f"response differs: {s}" for s in shape]
    else:
        tally["shapes_equal"] += 1
    row = {"name": name, "tokens": len(decision.prepared.ids), "route": decision.route, "dlogit": 0.0, "dp": 0.0, "agree": 0,
           "fields": len(fields), "margin": math.inf, "forward_ms": decision.timings["forward_ms"]}
    for i, f in enumerate(fields):
        at = f"{name}:{f}"
        want_logits = [float(x) for x in gold["logits"][f]]
        ours = [float(x) for x in decision.logits[i]] if i < len(decision.logits) else []
        if len(ours) != len(want_logits):
            tally["failures"].append(f"{at}: {len(ours)} logits, gold {len(want_logits)}")
            row["dlogit"] = math.nan
            continue
        margin = top2_margin(np.asarray(want_logits, dtype=np.float32))
        row["margin"] = min(row["margin"], margin)
        dl = 0.0
        for a, b in zip(ours, want_logits):
            d = abs(a - b)
            dl = _worst(dl, d)
            tally["sum_dlogit"] += d
            tally["logits"] += 1
        answer, want = decision.response["answers"].get(f, {}), gold["response"]["answers"][f]
        p, q = answer.get("probabilities"), want.get("probabilities")
        dp = math.nan
        if isinstance(p, dict) and isinstance(q, dict) and len(p) == len(q):
            dp = 0.0
            for key, pv in p.items():
                dp = _worst(dp, abs(pv - q[key]) if isinstance(q.get(key), float) and isinstance(pv, float) else math.nan)
        if not dp <= MAX_DP:   # a NaN fails
            tally["failures"].append(f"{at}: |dp| = {dp:.5f}, above {MAX_DP}")
        if math.isnan(dl):
            tally["failures"].append(f"{at}: NaN logit difference")
        row["dlogit"], row["dp"] = _worst(row["dlogit"], dl), _worst(row["dp"], dp)
        for slot, value in (("max_dlogit", dl), ("max_dp", dp)):
            if not math.isnan(tally[slot][0]) and (math.isnan(value) or value > tally[slot][0]):
                tally[slot] = (value, at)
        if answer.get("decision") == want.get("decision") and answer.get("choice") == want.get("choice"):
            row["agree"] += 1
        else:
            flip = f"{at}: {answer.get('decision')!r}, gold {want.get('decision')!r} (gold top-2 margin {margin:.4f})"
            if margin >= MARGIN or math.isnan(margin):
                tally["failures"].append(f"decision differs at {flip}")
            else:
                tally["small_flips"].append(flip)
    tally["fields"] += len(fields)
    tally["agree"] += row["agree"]
    tally["forward_ms"].append(row["forward_ms"])
    if row["route"] != "full":
        tally["snapshot"] += 1
    return row


def new_tally() -> dict:
    return {"requests": 0, "fields": 0, "agree": 0, "small_flips": [], "prompts_equal": 0, "shapes_equal": 0, "snapshot": 0,
            "max_dlogit": (0.0, "-"), "max_dp": (0.0, "-"), "sum_dlogit": 0.0, "logits": 0, "forward_ms": [], "failures": []}


def check(decide, gold: Path, requests: Path) -> tuple[bool, list]:
    """Runs every gold request through `decide(request_json) -> Decision` (DecisionEngine.decide); returns (pass, lines):
    the table and the summary of check.rs:270-343."""
    found = cases(gold, requests)
    lines = [f"{len(found)} gold requests from {gold}, requests from {requests}",
             f"criteria: decisions agree wherever the gold top-2 logit margin is >= {MARGIN}; calibrated |dp| <= {MAX_DP}; "
             "prompts and response envelopes identical", "",
             f"{'request':<18} {'tokens':>6}  {'route':<11}  {'max|dlogit|':>11}  {'max|dp|':>9}  {'decisions':>9}  {'gold margin':>11}  {'forward ms':>10}"]
    t = new_tally()
    for name, gold_path, request_path in found:
        gold_obj = json.loads(Path(gold_path).read_text())
        t["requests"] += 1
        try:
            d = decide(Path(request_path).read_text())
        except Exception as e:   # the engine refused or failed the request: a failure of the check, not of the run
            lines.append(f"{name:<18} error: {e}")
            t["failures"].append(f"{name}: the engine refused or failed the request: {e}")
            continue
        r = compare(name, d, gold_obj, t)
        lines.append(f"{name:<18} {r['tokens']:>6}  {r['route']:<11}  {r['dlogit']:>11.4f}  {r['dp']:>9.5f}  {r['agree']:>4}/{r['fields']:<4}  "
                     f"{r['margin']:>11.3f}  {r['forward_ms']:>10.1f}")
    ok = not t["failures"]
    lines.append("")
    if not ok:
        lines += ["failures:"] + [f"  {f}" for f in t["failures"]]
    ms = t["forward_ms"]
    lines += [f"summary: {t['requests']} requests, {t['fields']} fields: {'PASS' if ok else 'FAIL'}",
              f"  prompts identical to the gold's (ids, logit rows, fields, candidates): {t['prompts_equal']}/{t['requests']}",
              f"  responses with the gold's keys, key order, strings, ints and calibration (backend, timing, other floats aside): "
              f"{t['shapes_equal']}/{t['requests']}",
              f"  decisions agree: {t['agree']}/{t['fields']}; flips below the {MARGIN} gold margin (allowed): {'; '.join(t['small_flips']) or 'none'}",
              f"  max |dlogit| {t['max_dlogit'][0]:.4f} at {t['max_dlogit'][1]}; mean |dlogit| {t['sum_dlogit'] / max(t['logits'], 1):.4f} over {t['logits']} logits",
              f"  max |dp| {t['max_dp'][0]:.5f} at {t['max_dp'][1]} (tolerance {MAX_DP})",
              f"  route: from the prefix snapshot (or a cached state) {t['snapshot']}/{t['requests']}; forward mean "
              f"{sum(ms) / max(len(ms), 1):.1f} ms, max {max(ms, default=0.0):.1f} ms"]
    return ok, lines


def main():
    import argparse

    from . import prompt
    from .decision import DecisionEngine
    from .weight_files import open_engine

    ap = argparse.ArgumentParser(description="decide check: every gold request through the engine, against the fp32 gold files")
    ap.add_argument("--weights", required=True, help="a converted weight directory (decide-weights-v1)")
    ap.add_argument("--tokenizer", required=True, help="the checkpoint's tokenizer.json")
    ap.add_argument("--gold", required=True, help="directory of <set>/<name>.json gold files")
    ap.add_argument("--requests", required=True, help="directory of <set>/<name>.json requests")
    a = ap.parse_args()
    eng = open_engine(a.weights, max_rows=prompt.MAX_LENGTH, max_seqs=1, max_answers=16, max_cand=prompt.MAX_OPTIONS)
    de = DecisionEngine(eng, prompt.Tokenizer.from_file(a.tokenizer))
    ok, lines = check(de.decide, Path(a.gold), Path(a.requests))
    print("\n".join(lines))
    eng.close()
    raise SystemExit(0 if ok else 1)


if __name__ == "__main__":
    main()
