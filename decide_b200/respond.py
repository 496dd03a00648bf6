"""From candidate logits to the response a client receives: the reference's post-logit path
(crates/decide-engine/src/head.rs:45-141 softmax / calibration / decision, head.rs:154-172 `fields`,
head.rs:226-297 `respond_from`), which restates InternLM's `DecisionEngine.predict` from the logits on.

Everything here is host-side and exact by construction rather than by tolerance: softmax in f32,
temperature scaling (T = 1.99241824) in f64 through logs with Python's compensated sum, decision =
the largest calibrated probability with ties to the smaller label, floats printed as Python prints
them (`json.dumps` of this module's dict IS the reference's byte sequence, which its Rust side has to
imitate with a Python-float formatter). Key order follows the reference: type, probabilities,
confidence, the kind's own keys, source, decision; then usage, timing, calibration, model, backend.

The request side (JSON -> prompt -> token ids -> answer rows and candidate ids, crates/decide-prompt)
needs the tokenizer's data, which is not available here; a caller supplies each field's kind and
options (`Field`) together with the logits the engine returned for its candidates.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

TEMPERATURE = 1.99241824   # crates/decide-engine/src/config.rs:34
MODEL = "Intern-Decision-4B"
BACKEND = "decide-cuda"    # the reference's is "decide-metal" (head.rs:23), InternLM's "hf"


class HeadError(ValueError):
    """What the reference raises after its forward pass (same messages), or logits that do not fit the request."""


@dataclass
class Field:
    """One question of a request: its name, kind ("choice" | "score" | "noul") and its options in candidate order
    as (value, text) pairs; the text is the legend of a score option and unused otherwise."""
    name: str
    kind: str
    options: list = field(default_factory=list)


def softmax(logits) -> list:
    """head.rs:45-50: max, exp(x - max), sum, divide, all in f32."""
    x = [np.float32(v) for v in logits]
    mx = max(x)
    exps = [np.exp(np.float32(v - mx), dtype=np.float32) for v in x]
    total = np.float32(0.0)
    for e in exps:
        total = np.float32(total + e)
    return [np.float32(e / total) for e in exps]


def py_sum(xs) -> float:
    """Python's sum() of floats (Neumaier-compensated since 3.12), spelled out so that the result does not depend on
    the interpreter that runs this module (head.rs:80-97 does the same for Rust)."""
    xs = list(xs)
    if not xs:
        return 0.0
    total, c = 0.0 + xs[0], 0.0
    for x in xs[1:]:
        t = total + x
        c += (total - t) + x if abs(total) >= abs(x) else (x - t) + total
        total = t
    if c != 0.0 and math.isfinite(c):
        total += c
    return total


def argmax(labels, probs) -> int:
    """head.rs:63-77: the label minimising (-p, label): the largest probability, ties to the smaller label."""
    if len(labels) != len(probs) or not labels:
        raise HeadError("labels and probabilities must pair up and be non-empty")
    best = 0
    for i in range(1, len(labels)):
        a, b = -probs[i], -probs[best]
        if (labels[i] < labels[best]) if a == b else (a < b):
            best = i
    return best


def scale_probabilities(labels, probs, temperature: float = TEMPERATURE) -> list:
    """head.rs:116-141: p_i^(1/T) renormalised, in f64, through logs; refuses what the reference refuses."""
    probs = [float(p) for p in probs]
    if not math.isfinite(temperature) or temperature <= 0.0:
        raise HeadError("Temperature must be finite and positive")
    if not probs or any((not math.isfinite(p)) or p < 0.0 or p > 1.0 for p in probs):
        raise HeadError("Invalid probability distribution")
    if abs(py_sum(probs) - 1.0) > 0.001:
        raise HeadError("Probabilities must sum to one")
    if temperature == 1.0:
        return probs
    logs = [math.log(p) if p != 0.0 else -math.inf for p in probs]
    mx = max(logs)
    weights = [math.exp((l - mx) / temperature) for l in logs]
    total = py_sum(weights)
    result = [w / total for w in weights]
    if argmax(labels, result) != argmax(labels, probs):
        raise HeadError("Floating-point temperature scaling changed argmax")
    return result


def heads(fields: list, logits: list) -> list:
    """head.rs:154-172: per field (calibrated probabilities in option order, decision index)."""
    if len(logits) != len(fields):
        raise HeadError(f"{len(logits)} logit rows for {len(fields)} fields")
    out = []
    for f, row in zip(fields, logits):
        if len(row) != len(f.options):
            raise HeadError(f"{len(row)} logits for the {len(f.options)} options of {f.name!r}")
        labels = [value for value, _ in f.options]
        probs = scale_probabilities(labels, [float(p) for p in softmax(row)])   # `.tolist()` widens each f32 to a Python float
        out.append((probs, argmax(labels, probs)))
    return out


def _json_float(x: float) -> float:
    if not math.isfinite(x):
        raise HeadError(f"the response would carry {x!r}, which JSON cannot (the reference emits it)")
    return x


def respond(fields: list, logits: list, input_tokens: int, inference_ms: float, backend: str = BACKEND) -> dict:
    """head.rs:186-297. `logits[i]` are field i's candidate logits in option order; `input_tokens` is the full prompt
    length (although the forward pass stops at the last answer row); `inference_ms` the forward time. The dict's key
    order is the reference's; `json.dumps(result)` is the response text."""
    answers = {}
    for f, (p, best) in zip(fields, heads(fields, logits)):
        label = f.options[best][0]
        answer = {"type": f.kind, "probabilities": {value: _json_float(pi) for (value, _), pi in zip(f.options, p)},
                  "confidence": _json_float(p[best])}
        if f.kind == "noul":
            yes = [i for i, (value, _) in enumerate(f.options) if value == "yes"]
            if not yes:
                raise HeadError(f"noul field {f.name!r} has no \"yes\" option")
            answer["noul"] = _json_float(p[yes[0]])
        elif f.kind == "score":
            terms = []
            for (value, _), pi in zip(f.options, p):
                try:
                    terms.append(float(value) * pi)
                except ValueError:
                    raise HeadError(f"could not convert string to float: {value!r}") from None
            answer["score"] = _json_float(py_sum(terms))
            answer["legend"] = {value: text for value, text in f.options}
        elif f.kind == "choice":
            answer["choice"] = label
        else:
            raise HeadError(f"unknown field kind {f.kind!r}")
        answer["source"] = "local"
        answer["decision"] = label
        answers[f.name] = answer
    count = len(answers)
    ms = inference_ms if not math.isfinite(inference_ms) else float(f"{inference_ms:.2f}")
    return {"answers": answers,
            "usage": {"input_tokens": int(input_tokens), "output_tokens": count, "decision_count": count},
            "timing": {"inference_ms": _json_float(ms)},
            "calibration": {"method": "temperature-scaling", "temperature": TEMPERATURE},
            "model": MODEL, "backend": backend}
