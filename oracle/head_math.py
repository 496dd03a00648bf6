"""CPU restatement of the reference's post-logit head (crates/decide-engine/src/head.rs:45-141).

TEST INFRASTRUCTURE ONLY (see oracle/cpu_ref.py). Plain Python loops, one function per Rust
function: f32 softmax (head.rs:45-50), Python's compensated float sum (head.rs:80-97), the argmax
with ties to the smaller label (head.rs:63-77) and f64 temperature scaling (head.rs:116-141).
Pinned by the 65 fields of the reference's 58 gold fixtures (tests/golden/head_kat.json).
"""
from __future__ import annotations

import math

import numpy as np

TEMPERATURE = 1.99241824  # crates/decide-engine/src/config.rs:34


def softmax(logits) -> list:
    """head.rs:45-50: max, exp(x - max), sum, divide, all in f32."""
    x = [np.float32(v) for v in logits]
    mx = max(x)
    exps = [np.exp(np.float32(v - mx), dtype=np.float32) for v in x]
    total = np.float32(0.0)
    for e in exps:
        total = np.float32(total + e)
    return [np.float32(e / total) for e in exps]


def argmax(labels, probs) -> int:
    """head.rs:63-77: min(labels, key=lambda l: (-probs[l], l))."""
    if len(labels) != len(probs) or not labels:
        raise ValueError("labels and probabilities must pair up and be non-empty")
    best = 0
    for i in range(1, len(labels)):
        key, best_key = -probs[i], -probs[best]
        less = labels[i] < labels[best] if key == best_key else key < best_key
        if less:
            best = i
    return best


def py_sum(xs) -> float:
    """head.rs:80-97: Python 3.12's sum() of floats, Neumaier-compensated."""
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


def scale_probabilities(labels, probs, temperature: float = TEMPERATURE) -> list:
    """head.rs:116-141, f64."""
    probs = [float(p) for p in probs]
    if not math.isfinite(temperature) or temperature <= 0.0:
        raise ValueError("Temperature must be finite and positive")
    if not probs or any((not math.isfinite(p)) or p < 0.0 or p > 1.0 for p in probs):
        raise ValueError("Invalid probability distribution")
    if abs(py_sum(probs) - 1.0) > 0.001:
        raise ValueError("Probabilities must sum to one")
    if temperature == 1.0:
        return probs
    logs = [math.log(p) if p != 0.0 else -math.inf for p in probs]
    mx = max(logs)
    weights = [math.exp((l - mx) / temperature) for l in logs]
    total = py_sum(weights)
    result = [w / total for w in weights]
    if argmax(labels, result) != argmax(labels, probs):
        raise ValueError("Floating-point temperature scaling changed argmax")
    return result


def calibrated(logits, labels=None, temperature: float = TEMPERATURE):
    """Logits -> (calibrated probabilities, decision index), the chain the parity metric uses."""
    labels = labels if labels is not None else [f"{i:04d}" for i in range(len(logits))]
    p = scale_probabilities(labels, [float(v) for v in softmax(logits)], temperature)
    return p, argmax(labels, p)
