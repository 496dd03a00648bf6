"""Extracts request known-answer cases from the reference's request and gold fixtures.

    python tests/golden/make_request_kat.py /root/reference

For every `tests/fixtures/gold/fp32/{core,calib}/*.json` with its request
`tests/fixtures/requests/{core,calib}/*.json` it records the request's `questions` object and what the
reference's Python pipeline (InternLM's inference.py through reference/gold.py) derived from the request:
the field order, the candidate token ids per field, the answer rows and the prompt length. Together with
the option legends of `response_kat.json` these pin decide_b200/prompt.py's validate_request, options and
compile_row (field order, option order, option values and descriptions); the prompt TEXT and its token ids
need the checkpoint's tokenizer.json, which is not available, and stay unpinned. The `state` of a request is
not recorded: only the text depends on it.
"""
import json
import sys
from pathlib import Path


def main(reference: str):
    fixtures = Path(reference) / "tests" / "fixtures"
    cases = []
    for path in sorted((fixtures / "gold" / "fp32").glob("*/*.json")):
        if path.name == "activation_audit.json":
            continue
        req = fixtures / "requests" / path.parent.name / path.name
        if not req.exists():
            continue
        g, r = json.loads(path.read_text()), json.loads(req.read_text())
        cases.append({"file": f"{path.parent.name}/{path.name}", "questions": r["questions"], "fields": g["fields"],
                      "candidate_ids": [g["candidate_ids"][f] for f in g["fields"]], "positions": g["positions"], "n_ids": len(g["input_ids"])})
    out = Path(__file__).with_name("request_kat.json")
    out.write_text(json.dumps({"source": "tests/fixtures/{requests,gold/fp32} of ezulabs/decide", "cases": cases}, separators=(",", ":"), ensure_ascii=False))
    print(f"{len(cases)} requests -> {out} ({out.stat().st_size} bytes)")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
