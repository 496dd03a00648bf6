"""Request JSON -> prompt -> ids (decide_b200/prompt.py) against what the reference's pipeline derived from its 58
request fixtures (tests/golden/request_kat.json, response_kat.json), the reference's validation messages
(crates/decide-prompt/src/request.rs:58-133), and a synthetic byte-level tokenizer for the stage that needs
tokenizer.json (the checkpoint's is not available: the prompt text and its ids are unpinned)."""
import json
from pathlib import Path

import pytest

from decide_b200 import prompt

GOLDEN = Path(__file__).parent / "golden"
REQUESTS = json.loads((GOLDEN / "request_kat.json").read_text())["cases"]
RESPONSES = {c["file"]: c for c in json.loads((GOLDEN / "response_kat.json").read_text())["cases"]}


def test_all_58_requests_are_held():
    assert len(REQUESTS) == 58 and all(c["file"] in RESPONSES for c in REQUESTS)


@pytest.mark.parametrize("case", REQUESTS, ids=[c["file"] for c in REQUESTS])
def test_fields_and_options_as_the_reference_derived_them(case):
    """Field order, option count, option values and descriptions (the response's legend), and one row per field."""
    row = prompt.validate_request({"state": "s", "questions": case["questions"]})
    c = prompt.compile_row(row)
    assert c.fields == case["fields"]
    assert [len(o) for o in c.options] == [len(ids) for ids in case["candidate_ids"]]
    assert len(case["positions"]) == len(c.fields)
    gold = RESPONSES[case["file"]]["fields"]
    for q, opts, want in zip(row.questions, c.options, gold):
        assert q.kind == want["kind"] and q.name == want["name"]
        assert [v for _, v, _ in opts] == [v for v, _ in want["options"]]
        for (_, _, desc), (_, legend) in zip(opts, want["options"]):
            if legend:
                assert desc == legend
        assert [s for s, _, _ in opts] == list(prompt.ANSWER_SYMBOLS[:len(opts)])


def test_candidate_symbols_are_one_table():
    """The reference gives field i the first n_i symbol ids of ONE table (tokenize.rs:120): every fixture's candidate ids
    are a prefix of the longest list seen."""
    longest = max((ids for c in REQUESTS for ids in c["candidate_ids"]), key=len)
    for c in REQUESTS:
        for ids in c["candidate_ids"]:
            assert ids == longest[:len(ids)]


def test_user_text_and_skeleton():
    req = {"state": {"note": "Charged twice — wants a refund", "amount": 12.50, "n": 3, "flags": [True, None]},
           "questions": {"team": {"type": "choice", "instructions": "Which team?", "criteria": {"billing": "Payments", "delivery": 7}},
                         "urgency": {"type": "score", "criteria": ["Low", "High"]},
                         "refund": {"type": "noul", "instructions": None, "criteria": {"YES": "asks for money back"}}}}
    c = prompt.compile_row(prompt.validate_request(req))
    assert c.user_text == (
        "Return one answer for every field using the supplied answer symbols.\n\n## State\n"
        '{\n  "note": "Charged twice — wants a refund",\n  "amount": 12.5,\n  "n": 3,\n  "flags": [\n    true,\n    null\n  ]\n}\n'
        "## Decision schema\n"
        "team: Which team?\n    A = billing: Payments\n    B = delivery: 7\n"
        "urgency: \n    A = 0: Low\n    B = 1: High\n"
        "refund: None\n    A = no: The answer is no (negative, or disagree with the claim).\n    B = yes: asks for money back")
    assert c.skeleton == '{\n    "team": "<decision>",\n    "urgency": "<decision>",\n    "refund": "<decision>"\n}'
    text = prompt.render(prompt.SYSTEM_PROMPT, c.user_text, c.skeleton)
    assert text.startswith(prompt.prefix_text()) and text.endswith('"refund": "<decision>"\n}<|im_end|>\n')
    assert "<|im_start|>assistant\n<think>\n\n</think>\n\n{" in text
    assert prompt.STATE_MARKER_TEXT in text


@pytest.mark.parametrize("request_,message", [
    ([1], "Supply a JSON object containing state and questions."),
    ({"questions": {}}, "Supply a JSON object containing state and questions."),
    ({"state": 1, "questions": {}}, "Supply 1–16 questions."),
    ({"state": 1, "questions": {str(i): {"type": "noul"} for i in range(17)}}, "Supply 1–16 questions."),
    ({"state": 1, "questions": {"": {"type": "noul"}}}, "Question names must be nonempty strings."),
    ({"state": 1, "questions": {"a": {"type": "rank"}}}, "Question type must be choice, score, or noul."),
    ({"state": 1, "questions": {"a": "noul"}}, "Question type must be choice, score, or noul."),
    ({"state": 1, "questions": {"a": {"type": "choice", "criteria": ["x"]}}}, "Choice criteria must be an object."),
    ({"state": 1, "questions": {"a": {"type": "score", "criteria": "x"}}}, "Score criteria must be a list or object."),
    ({"state": 1, "questions": {"a": {"type": "score", "criteria": {"one": "x"}}}}, "Score option keys must be finite numbers."),
    ({"state": 1, "questions": {"a": {"type": "score", "criteria": {"inf": "x"}}}}, "Score option keys must be finite numbers."),
    ({"state": 1, "questions": {"a": {"type": "score", "criteria": []}}}, "Supply 1–62 options."),
    ({"state": 1, "questions": {"a": {"type": "choice", "criteria": {str(i): "x" for i in range(63)}}}}, "Supply 1–62 options."),
    ({"state": "has <decision> inside", "questions": {"a": {"type": "noul"}}}, "Reserved decision marker appears in input evidence"),
    ({"state": 1, "images": "x.png", "questions": {"a": {"type": "noul"}}}, "Upload 1–8 images."),
    ({"state": 1, "images": ["x"] * 9, "questions": {"a": {"type": "noul"}}}, "Upload 1–8 images."),
    ({"state": 1, "images": ["x", ""], "questions": {"a": {"type": "noul"}}}, "Images must be nonempty local file paths."),
    ({"state": 1, "images": ["x.png"], "questions": {"a": {"type": "noul"}}}, "decide is text-only"),
    ({"state": 1, "questions": {"a": {"type": "noul", "instructions": ["x"]}}}, "decide accepts only strings, numbers, booleans or null"),
])
def test_refusals_carry_the_reference_messages(request_, message):
    with pytest.raises(prompt.RequestError, match=message):
        prompt.validate_request(request_)


def test_empty_images_are_ignored_and_score_keys_parse_like_python_floats():
    row = prompt.validate_request({"state": 1, "images": [], "questions": {"a": {"type": "score", "criteria": {"1e3": "k", " 2.5 ": "m", "1_0": "t"}}}})
    assert [v for v, _ in prompt.options(row.questions[0])] == ["1e3", " 2.5 ", "1_0"]


def test_json_errors():
    with pytest.raises(ValueError, match="request is not valid JSON"):
        prompt.prompt_text("{")
    with pytest.raises(prompt.RequestError, match="Exceeds the limit"):
        prompt.prompt_text('{"state": ' + "1" * 4301 + ', "questions": {"a": {"type": "noul"}}}')


def byte_level_tokenizer_file(path):
    """A tokenizer.json with the 256 byte-level symbols as its whole vocabulary, no merges, the NFC normalizer and the
    reference's added tokens: every character is its bytes' tokens, every added token one id."""
    import tokenizers
    from tokenizers import models, normalizers, pre_tokenizers

    alphabet = sorted(pre_tokenizers.ByteLevel.alphabet())
    tok = tokenizers.Tokenizer(models.BPE(vocab={ch: i for i, ch in enumerate(alphabet)}, merges=[]))
    tok.normalizer = normalizers.NFC()
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)   # the file's own; prompt.Tokenizer replaces it
    tok.add_special_tokens(["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", prompt.DECISION_TOKEN])
    tok.save(str(path))


def test_prepare_with_a_byte_level_tokenizer(tmp_path):
    """ids, the row before every decision marker, candidate ids per field, the prefix property the snapshot rests on, and
    the state marker the state cache looks for (tokenize.rs:99-125, template.rs:25-28, forward.rs:65-70)."""
    byte_level_tokenizer_file(tmp_path / "tokenizer.json")
    tok = prompt.Tokenizer.from_file(tmp_path / "tokenizer.json")
    req = {"state": {"text": "naïve café ☕"}, "questions": {"team": {"type": "choice", "criteria": {"a": "x", "b": "y", "c": "z"}}, "ok": {"type": "noul"}}}
    p = tok.prepare(json.dumps(req))
    assert len(p.positions) == 2 and [p.ids[i + 1] for i in p.positions] == [tok.marker] * 2
    assert p.positions == sorted(p.positions) and p.positions[0] > 0
    assert p.candidates == [tok.symbol_ids[:3], tok.symbol_ids[:2]] and len(set(tok.symbol_ids)) == 62
    prefix = tok.prefix_ids()
    assert p.ids[:len(prefix)] == prefix and len(prefix) < p.positions[0]
    marker = tok.state_marker_ids()
    at = [i for i in range(len(prefix), p.positions[0]) if p.ids[i:i + len(marker)] == marker]
    assert len(at) == 1, "the state marker occurs once between the prefix and the first answer row"
    # the pre-tokenizer is the one the reference runs, as its fixture of the tokenizer pipeline records it
    mine = json.loads(tok.inner.to_str())["pre_tokenizer"]
    assert mine["pretokenizers"][0]["pattern"] == {"Regex": prompt.REFERENCE_PRETOKENIZE_REGEX}
    assert mine["pretokenizers"][0]["behavior"] == "Isolated" and mine["pretokenizers"][0]["invert"] is False
    assert mine["pretokenizers"][1] == {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": False}
    with pytest.raises(ValueError, match="truncation is forbidden"):
        tok.prepare(json.dumps(req), max_length=50)
