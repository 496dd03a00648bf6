"""Extracts response known-answer cases from the reference's gold fixtures.

    python tests/golden/make_response_kat.py /root/reference

For every `tests/fixtures/gold/fp32/{core,calib}/*.json` it records what the response builder needs
(each field's kind, option values and legend texts in order, the fp32 gold logits, the prompt
length, the forward time) and the `response` object the reference's Python pipeline produced from
them (reference/gold.py:66-95 and InternLM's DecisionEngine.predict). tests/test_respond.py checks
decide_b200/respond.py against these byte for byte; no model weights are involved.
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
        fields = []
        for name in g["fields"]:
            ans = g["response"]["answers"][name]
            legend = ans.get("legend", {})
            fields.append({"name": name, "kind": ans["type"], "options": [[v, legend.get(v, "")] for v in ans["probabilities"]]})
        cases.append({"file": f"{path.parent.name}/{path.name}", "fields": fields, "logits": [g["logits"][f] for f in g["fields"]],
                      "input_tokens": g["response"]["usage"]["input_tokens"], "inference_ms": g["seconds"] * 1e3, "response": g["response"]})
    out = Path(__file__).with_name("response_kat.json")
    out.write_text(json.dumps({"source": "tests/fixtures/gold/fp32 of ezulabs/decide", "cases": cases}, separators=(",", ":")))
    print(f"{len(cases)} responses -> {out} ({out.stat().st_size} bytes)")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
