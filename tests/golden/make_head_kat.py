"""Extracts the post-logit head known-answer vectors from the reference's gold fixtures.

Run once in a checkout that has the reference mounted:
    python tests/golden/make_head_kat.py /root/reference
For every field of every `tests/fixtures/gold/fp32/{core,calib}/*.json` it records the fp32 gold
logits, the labels in dict order, the calibrated probabilities and the decision that the
reference's Python pipeline produced from them (reference/gold.py:66-95 response_from_logits:
softmax in f32, temperature scaling 1.99241824 in f64, argmax with ties to the smaller label).
The result, tests/golden/head_kat.json, is what tests/test_head.py checks the restated head math
against; it needs no model weights.
"""
import json
import sys
from pathlib import Path


def main(reference: str):
    root = Path(reference) / "tests" / "fixtures" / "gold" / "fp32"
    cases = []
    for path in sorted(root.glob("*/*.json")):
        if path.name == "activation_audit.json":
            continue
        g = json.loads(path.read_text())
        temperature = g["response"]["calibration"]["temperature"]
        for field in g["fields"]:
            ans = g["response"]["answers"][field]
            labels = list(ans["probabilities"].keys())
            cases.append({
                "file": f"{path.parent.name}/{path.name}", "field": field, "temperature": temperature,
                "logits": g["logits"][field], "labels": labels,
                "probabilities": [ans["probabilities"][l] for l in labels], "decision": ans["decision"],
            })
    out = Path(__file__).with_name("head_kat.json")
    out.write_text(json.dumps({"source": "tests/fixtures/gold/fp32 of ezulabs/decide", "cases": cases}, indent=0))
    print(f"{len(cases)} fields from {len(set(c['file'] for c in cases))} files -> {out}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
