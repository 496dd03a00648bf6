"""Request JSON in, response JSON out: the reference's `Engine` (crates/decide-engine/src/engine.rs:110-265) over the
CUDA prefill. `DecisionEngine.decide` is InternLM's `DecisionEngine.predict`: prepare the prompt (prompt.py), run the
prefill for the rows before each decision marker (engine.py), turn the candidate logits into the response (respond.py).

At construction the constant head of every prompt is run once and kept as the prefix snapshot, and the state cache is
told which token ids end a request's state (engine.rs:160-185): a first request about a state runs from the snapshot
and leaves the state in the cache, other questions about the same state run only the rows after it.
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass

import numpy as np

from . import prompt, respond
from .synth import Batch


@dataclass
class Decision:
    """engine.rs:112-127."""
    response: dict
    prepared: prompt.Prepared
    logits: list            # per field, its candidates' logits in option order
    route: str              # "full" | "snapshot" | "state_cache"
    rows: int               # rows the prefill computed
    timings: dict           # tokenize_ms, forward_ms, head_ms

    def text(self) -> str:
        """The response as the client receives it."""
        return json.dumps(self.response, ensure_ascii=False)


def fields_of(prepared: prompt.Prepared) -> list:
    """The response builder's view of a prepared request: each field's kind and (value, description) options."""
    return [respond.Field(q.name, q.kind, [(value, text) for _, value, text in opts])
            for q, opts in zip(prepared.row.questions, prepared.compiled.options)]


class DecisionEngine:
    def __init__(self, engine, tokenizer: prompt.Tokenizer, snapshot: bool = True, state_entries: int | None = None):
        """`engine`: an `Engine` (e.g. `weight_files.open_engine(directory)`) created with room for one request
        (`max_rows` >= the longest prompt, `max_answers` >= 16, `max_cand` >= the most options of a field)."""
        self.engine, self.tokenizer = engine, tokenizer
        if snapshot:
            engine.build_snapshot(np.asarray(tokenizer.prefix_ids(), dtype=np.uint32))
            engine.set_state_marker(np.asarray(tokenizer.state_marker_ids(), dtype=np.uint32))
        if state_entries is not None:
            engine.set_state_cache(state_entries)

    def prepare(self, request_json: str) -> prompt.Prepared:
        return self.tokenizer.prepare(request_json, prompt.MAX_LENGTH)

    def logits(self, prepared: prompt.Prepared) -> list:
        """Engine::logits (engine.rs:226-230): the prompt's ids with the answers at `prepared.positions`."""
        n, width = len(prepared.positions), self.engine.max_cand
        if max(len(c) for c in prepared.candidates) > width:
            raise ValueError(f"a field has {max(len(c) for c in prepared.candidates)} options; the engine was created for {width}")
        cand = np.zeros((n, width), dtype=np.uint32)
        for i, c in enumerate(prepared.candidates):
            cand[i, :len(c)] = c
        ncand = np.array([len(c) for c in prepared.candidates], dtype=np.uint32)
        ids = np.asarray(prepared.ids, dtype=np.uint32)
        batch = Batch(ids, np.array([0, len(ids)], dtype=np.uint32), np.asarray(prepared.positions, dtype=np.uint32), cand, ncand)
        out = self.engine.logits(batch)
        return [out[i, :len(c)].tolist() for i, c in enumerate(prepared.candidates)]

    def decide(self, request_json: str) -> Decision:
        """Engine::decide (engine.rs:236-265)."""
        t0 = time.perf_counter()
        prepared = self.prepare(request_json)
        t1 = time.perf_counter()
        logits = self.logits(prepared)
        t2 = time.perf_counter()
        forward_ms = 1e3 * (t2 - t1)
        response = respond.respond(fields_of(prepared), logits, len(prepared.ids), forward_ms)
        t3 = time.perf_counter()
        return Decision(response, prepared, logits, self.engine.last_route, self.engine.resident_rows - self.engine.last_start,
                        {"tokenize_ms": 1e3 * (t1 - t0), "forward_ms": forward_ms, "head_ms": 1e3 * (t3 - t2)})
