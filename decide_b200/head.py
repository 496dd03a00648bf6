"""Post-logit head on the host: softmax, temperature scaling, decision.

The two functions of the reference's head that the parity metric needs
(crates/decide-engine/src/head.rs:45-50 softmax in f32; head.rs:116-141 temperature scaling in f64
with T = 1.99241824, config.rs:34; head.rs:63-77 argmax with ties to the smaller label), vectorised
over answer rows with numpy. The response JSON, labels and question types of head.rs:154-297 are
outside the hot path.
"""
from __future__ import annotations

import numpy as np

TEMPERATURE = 1.99241824


def softmax_f32(logits: np.ndarray) -> np.ndarray:
    """Row-wise softmax in f32 over the last axis."""
    x = np.asarray(logits, dtype=np.float32)
    e = np.exp(x - x.max(axis=-1, keepdims=True), dtype=np.float32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)


def scale_probabilities(probs: np.ndarray, temperature: float = TEMPERATURE) -> np.ndarray:
    """p_i^(1/T) renormalised, in f64, computed through logs as the reference does."""
    if not np.isfinite(temperature) or temperature <= 0:
        raise ValueError("Temperature must be finite and positive")
    p = np.asarray(probs, dtype=np.float64)
    if p.size == 0 or not np.isfinite(p).all() or (p < 0).any() or (p > 1).any():
        raise ValueError("Invalid probability distribution")
    if (np.abs(p.sum(axis=-1) - 1.0) > 0.001).any():
        raise ValueError("Probabilities must sum to one")
    if temperature == 1.0:
        return p
    with np.errstate(divide="ignore"):
        logs = np.where(p != 0.0, np.log(p), -np.inf)
    w = np.exp((logs - logs.max(axis=-1, keepdims=True)) / temperature)
    return w / w.sum(axis=-1, keepdims=True)


def decide(logits: np.ndarray, ncand=None, temperature: float = TEMPERATURE):
    """logits [n, max_cand] (+ candidates used per row) -> (calibrated probabilities [n, max_cand] with
    zeros past ncand, decisions [n]). Ties go to the lower candidate index."""
    logits = np.asarray(logits, dtype=np.float32)
    n, mc = logits.shape
    ncand = np.full(n, mc) if ncand is None else np.asarray(ncand)
    probs = np.zeros((n, mc), dtype=np.float64)
    dec = np.zeros(n, dtype=np.int64)
    for i in range(n):
        c = int(ncand[i])
        probs[i, :c] = scale_probabilities(softmax_f32(logits[i, :c]), temperature)
        dec[i] = int(np.argmax(probs[i, :c]))  # first maximum = lowest index on ties
    return probs, dec
