"""Request JSON -> prompt text -> token ids, answer rows and candidate ids: the stage in front of the prefill
(crates/decide-prompt/src/*.rs, which restates InternLM's inference.py in Rust; here Python's own `json`, `str()` and
float formatting ARE the semantics the reference emulates).

    request.rs:58-133   validate_request   same checks, same messages
    request.rs:139-172  options            (value, description) per option, in order
    compile.rs:21-50    compile_row        user text (preamble, state as indented JSON, decision schema) + answer skeleton
    template.rs:8-28    render, prefix_text the chat template for [system, user, assistant skeleton], thinking off
    tokenize.rs:49-127  Tokenizer          tokenizer.json with the reference's pre-tokenizer; ids, the row before every
                                           decision marker, the candidate symbol ids per field

The tokenizer's data (tokenizer.json of the checkpoint) is not part of this repository: `Tokenizer.from_file` takes its
path. Everything up to the text works without it.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field

ANSWER_SYMBOLS = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789"   # request.rs:6
MAX_OPTIONS = 62
MAX_LENGTH = 8192                                                                     # the reference's max_length (engine.rs:218-221)
SYSTEM_PROMPT = ("You are a careful decision assistant. Use the state and decision schema in the user message to make the requested "
                 "decisions. For every field, choose exactly one answer symbol (e.g. A, B, C, ...) from its listed options and return one "
                 "valid JSON object mapping each field name to its chosen symbol. Use the field names and symbols exactly as given. Do not "
                 "include explanations, Markdown, or extra text.")                   # compile.rs:7
DECISION_TOKEN = "<decision>"
USER_PREAMBLE = "Return one answer for every field using the supplied answer symbols.\n\n## State\n"
STATE_MARKER_TEXT = "## Decision schema\n"   # the line that ends a request's state (forward.rs:65-70)

# The split regex the reference runs (tokenize.rs:56-57): the original Qwen2 one, without \p{M}.
REFERENCE_PRETOKENIZE_REGEX = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"


class RequestError(ValueError):
    """A request the reference rejects (same message), or one decide refuses where the reference would not."""


@dataclass
class Question:
    name: str
    kind: str                      # "choice" | "score" | "noul"
    instructions: object = None    # None when absent: printed as '' (request.rs:21-22)
    criteria: object = None
    has_instructions: bool = False


@dataclass
class Row:
    state: object
    questions: list[Question]


@dataclass
class Compiled:
    user_text: str
    skeleton: str
    fields: list[str]
    options: list[list[tuple[str, str, str]]]   # per field: (symbol, option value, description)


@dataclass
class Prepared:
    text: str
    ids: list[int]
    positions: list[int]            # the row before each decision marker, one per field
    candidates: list[list[int]]     # candidate symbol token ids per field, in option order
    row: Row
    compiled: Compiled = field(repr=False, default=None)


def str_of(v) -> str:
    """Python's str() of a JSON scalar; lists and dicts are refused as decide refuses them (pystr.rs:21-35)."""
    if isinstance(v, (list, dict)):
        raise RequestError("decide accepts only strings, numbers, booleans or null as instructions and option descriptions "
                           "(the reference would print a Python repr)")
    return str(v)


def _finite_number(text: str) -> bool:
    try:
        x = float(text)
    except ValueError:
        return False
    return x == x and x not in (float("inf"), float("-inf"))


def options(q: Question) -> list[tuple[str, str]]:
    """`_options(question)`: (value, description) in order (request.rs:139-172)."""
    c = q.criteria
    if q.kind in ("choice", "score") and isinstance(c, dict):
        return [(k, str_of(v)) for k, v in c.items()]
    if q.kind == "score" and isinstance(c, list):
        return [(str(i), str_of(v)) for i, v in enumerate(c)]
    if q.kind == "noul":
        d = c if isinstance(c, dict) else {}

        def pick(keys, default):
            for k, v in d.items():
                if k.lower() in keys:
                    return str_of(v)
            return default

        yes = pick(("yes", "true", "1"), "The answer is yes (affirmative, or align with the claim).")
        no = pick(("no", "false", "0"), "The answer is no (negative, or disagree with the claim).")
        return [("no", no), ("yes", yes)]
    raise RequestError("choice criteria must be an object" if q.kind == "choice" else "score criteria must be a list or object")


def compile_row(row: Row) -> Compiled:
    """InternLM's compile_row: the user message and the JSON answer skeleton (compile.rs:21-50)."""
    schema, fields, per_field = [], [], []
    for q in row.questions:
        opts = options(q)
        if len(opts) > MAX_OPTIONS:
            raise RequestError(f"At most {MAX_OPTIONS} single-token answer symbols are supported")
        instructions = str_of(q.instructions) if q.has_instructions else ""
        schema.append(f"{q.name}: {instructions}")
        entries = []
        for symbol, (value, description) in zip(ANSWER_SYMBOLS, opts):
            schema.append(f"    {symbol} = {value}: {description}")
            entries.append((symbol, value, description))
        fields.append(q.name)
        per_field.append(entries)
    state = json.dumps(row.state, ensure_ascii=False, indent=2)
    user_text = f"{USER_PREAMBLE}{state}\n## Decision schema\n" + "\n".join(schema)
    if DECISION_TOKEN in user_text:
        raise RequestError("Reserved decision marker appears in input evidence")
    skeleton = json.dumps({f: DECISION_TOKEN for f in fields}, ensure_ascii=False, indent=4)
    return Compiled(user_text, skeleton, fields, per_field)


def validate_request(request) -> Row:
    """InternLM's validate_request with its messages (request.rs:58-133)."""
    if not isinstance(request, dict) or "state" not in request:
        raise RequestError("Supply a JSON object containing state and questions.")
    images = request.get("images") or None
    if images is not None:
        if not isinstance(images, list) or len(images) > 8:
            raise RequestError("Upload 1–8 images.")
        if not all(isinstance(i, str) and i for i in images):
            raise RequestError("Images must be nonempty local file paths.")
    questions = request.get("questions")
    if not isinstance(questions, dict) or not 1 <= len(questions) <= 16:
        raise RequestError("Supply 1–16 questions.")
    out = []
    for name, q in questions.items():
        if not name:
            raise RequestError("Question names must be nonempty strings.")
        kind = q.get("type") if isinstance(q, dict) else None
        if not isinstance(kind, str) or kind not in ("choice", "score", "noul"):
            raise RequestError("Question type must be choice, score, or noul.")
        criteria = q.get("criteria")
        if kind == "choice" and not isinstance(criteria, dict):
            raise RequestError("Choice criteria must be an object.")
        if kind == "score":
            if isinstance(criteria, dict):
                if not all(_finite_number(k) for k in criteria):
                    raise RequestError("Score option keys must be finite numbers.")
            elif not isinstance(criteria, list):
                raise RequestError("Score criteria must be a list or object.")
        if kind != "noul":
            n = len(criteria) if isinstance(criteria, (list, dict)) else 0
            if not 1 <= n <= MAX_OPTIONS:
                raise RequestError(f"Supply 1–{MAX_OPTIONS} options.")
        out.append(Question(name, kind, q.get("instructions"), criteria, "instructions" in q))
    row = Row(request["state"], out)
    compile_row(row)   # the reference validates by compiling
    if images is not None:
        raise RequestError("decide is text-only: remove `images` (the reference would accept them).")
    return row


def render(system: str, user: str, assistant: str) -> str:
    """The checkpoint's chat template for [system, user, assistant skeleton], no generation prompt, thinking off; every
    content is stripped as Jinja's `|trim` does (template.rs:8-23)."""
    content, reasoning = assistant.strip(), ""
    if "</think>" in content:
        before = content.split("</think>")[0].rstrip("\n")
        reasoning = before.split("<think>")[-1].lstrip("\n")
        content = content.split("</think>")[-1].lstrip("\n")
    return (f"<|im_start|>system\n{system.strip()}<|im_end|>\n<|im_start|>user\n{user.strip()}<|im_end|>\n"
            f"<|im_start|>assistant\n<think>\n{reasoning.strip()}\n</think>\n\n{content}<|im_end|>\n")


def prefix_text() -> str:
    """The constant head of every prompt: everything through "## State\\n" (template.rs:25-28). Its ids are what
    Engine.build_snapshot takes."""
    return f"<|im_start|>system\n{SYSTEM_PROMPT}<|im_end|>\n<|im_start|>user\n{USER_PREAMBLE}"


def prompt_text(request_json: str) -> tuple[str, Row, Compiled]:
    """Request JSON text -> (prompt text, validated row, compiled row); no tokenizer needed."""
    try:
        request = json.loads(request_json)   # raises the reference's ValueError for an int literal of more than 4300 digits too
    except json.JSONDecodeError as e:
        raise ValueError(f"request is not valid JSON: {e}") from None
    except ValueError as e:
        raise RequestError(str(e)) from None
    row = validate_request(request)
    compiled = compile_row(row)
    return render(SYSTEM_PROMPT, compiled.user_text, compiled.skeleton), row, compiled


class Tokenizer:
    """tokenizer.json with the pre-tokenizer the reference actually runs (tokenize.rs:49-97): vocabulary, merges, the NFC
    normalizer and the added tokens are the file's; the split regex is the original Qwen2 one."""

    def __init__(self, inner):
        from tokenizers import Regex, pre_tokenizers

        self.inner = inner
        inner.pre_tokenizer = pre_tokenizers.Sequence([
            pre_tokenizers.Split(Regex(REFERENCE_PRETOKENIZE_REGEX), behavior="isolated", invert=False),
            pre_tokenizers.ByteLevel(add_prefix_space=False, trim_offsets=True, use_regex=False),
        ])
        self.marker = inner.token_to_id(DECISION_TOKEN)
        if self.marker is None:
            raise ValueError(f"tokenizer lacks {DECISION_TOKEN}")
        self.symbol_ids = []
        for c in ANSWER_SYMBOLS:
            ids = inner.encode(c, add_special_tokens=False).ids
            if len(ids) != 1:
                raise ValueError("Candidate symbols must each encode to a single token")
            self.symbol_ids.append(ids[0])

    @classmethod
    def from_file(cls, path) -> "Tokenizer":
        import tokenizers

        return cls(tokenizers.Tokenizer.from_file(str(path)))

    def encode(self, text: str) -> list[int]:
        return self.inner.encode(text, add_special_tokens=False).ids

    def prefix_ids(self) -> list[int]:
        return self.encode(prefix_text())

    def state_marker_ids(self) -> list[int]:
        """The ids of the line that ends a request's state, for Engine.set_state_marker (forward.rs:65-70, 765-772)."""
        return self.encode(STATE_MARKER_TEXT)

    def prepare(self, request_json: str, max_length: int = MAX_LENGTH) -> Prepared:
        """Request JSON -> ids, answer rows, candidates (Tokenizer::prepare, tokenize.rs:99-125)."""
        text, row, compiled = prompt_text(request_json)
        ids = self.encode(text)
        if len(ids) > max_length:
            raise ValueError(f"Example has {len(ids)} tokens, above {max_length}; truncation is forbidden")
        positions = [i - 1 for i, t in enumerate(ids) if t == self.marker]
        if len(positions) != len(compiled.fields) or -1 in positions:
            raise ValueError("Decision marker count or position mismatch")
        candidates = [self.symbol_ids[:len(o)] for o in compiled.options]
        return Prepared(text, ids, positions, candidates, row, compiled)
