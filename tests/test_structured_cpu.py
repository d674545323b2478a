"""Structured output: the regex engine against Python's ``re``, JSON-schema lowering against ``json`` and a
hand-written validator, token masks against brute force, and constrained generation end to end."""
import json
import random
import re
import zlib

import pytest

from tokenweave_b200.engine.structured import (DFA, GuidedFSM, RegexError, TokenTrie, json_schema_to_regex)

PATTERNS = [
    r"abc", r"a|bc|d", r"(ab)*c", r"a+b?c*", r"[a-c]{2,4}x", r"[^abc]+", r"\d{3}-\d{4}", r"(a|b)(c|d){0,2}e",
    r"x{3}", r"x{2,}", r"(?:ab|cd)+", r"\w+@\w+\.(com|org)", r"[A-Za-z_][A-Za-z0-9_]*", r"a.c", r"\s*-?\d+(\.\d+)?\s*",
    r"(0|[1-9][0-9]*)", r"[\d.]+", r"[a\-z]+", r"\(\d+\)", r"(a|ab)(c|bcd)", r"(a*)*b", r"é+|ü", r"[é-ë]x", r"^ab$",
    r"(yes|no|maybe)( (yes|no|maybe))*", r"\"([^\"\\]|\\.)*\"", r"a{0}b", r"a??b", r"a+?b",
]


@pytest.mark.parametrize("pattern", PATTERNS)
def test_regex_engine_agrees_with_re(pattern):
    dfa = DFA(pattern)
    rx = re.compile(pattern, re.ASCII)          # \w \d \s are ASCII classes in the engine
    rng = random.Random(zlib.crc32(pattern.encode()))
    alphabet = sorted(set(c for c in pattern if c.isalnum() or c in " .-@_\"\\") | set("abcdxyz019 -.@_(éëêü"))
    samples = {""}
    for _ in range(1500):
        samples.add("".join(rng.choice(alphabet) for _ in range(rng.randrange(0, 9))))
    # strings grown from the automaton itself, so that accepting paths are well represented
    for _ in range(300):
        s, out = 0, bytearray()
        for _ in range(rng.randrange(1, 30)):
            nxt = [b for b in range(256) if dfa.step(s, b) >= 0]
            if not nxt:
                break
            b = rng.choice(nxt)
            out.append(b)
            s = dfa.step(s, b)
            if dfa.accepting[s]:            # every accepted prefix on the way is a sample too
                try:
                    samples.add(out.decode("utf-8"))
                except UnicodeDecodeError:
                    pass
        try:
            samples.add(out.decode("utf-8"))
        except UnicodeDecodeError:
            pass
    agree_accept = 0
    for text in samples:
        want = rx.fullmatch(text) is not None
        assert dfa.fullmatch(text) == want, (pattern, text)
        agree_accept += want
    assert agree_accept > 0, f"no accepted sample for {pattern}"


def test_bad_patterns_are_refused():
    for bad in [r"(ab", r"a)", r"*a", r"a{2,1}", r"(?=a)b", r"a\bb", r"[abc", r"\p{L}"]:
        with pytest.raises((RegexError, ValueError)):
            DFA(bad)


SCHEMA = {
    "type": "object",
    "properties": {
        "name": {"type": "string", "maxLength": 8},
        "age": {"type": "integer"},
        "tags": {"type": "array", "items": {"enum": ["a", "b", "c d"]}, "minItems": 1, "maxItems": 3},
        "score": {"type": ["number", "null"]},
        "address": {"$ref": "#/$defs/addr"},
        "nick": {"type": "string"},
    },
    "required": ["name", "age", "tags", "address"],
    "$defs": {"addr": {"type": "object", "properties": {"zip": {"type": "string", "pattern": "[0-9]{5}"},
                                                        "ok": {"type": "boolean"}}, "required": ["zip"]}},
}


def _conforms(v) -> bool:
    if not isinstance(v, dict) or not {"name", "age", "tags", "address"} <= set(v) or set(v) - set(SCHEMA["properties"]):
        return False
    ok = isinstance(v["name"], str) and len(v["name"]) <= 8 and isinstance(v["age"], int) and not isinstance(v["age"], bool)
    ok &= isinstance(v["tags"], list) and 1 <= len(v["tags"]) <= 3 and all(t in ("a", "b", "c d") for t in v["tags"])
    ok &= v.get("score") is None or (isinstance(v["score"], (int, float)) and not isinstance(v["score"], bool))
    a = v["address"]
    ok &= isinstance(a, dict) and re.fullmatch("[0-9]{5}", a.get("zip", "")) is not None and set(a) <= {"zip", "ok"}
    ok &= isinstance(a.get("ok", True), bool) and isinstance(v.get("nick", ""), str)
    return bool(ok)


def test_json_schema_regex_accepts_conforming_documents_only():
    dfa = DFA(json_schema_to_regex(SCHEMA))
    good = [
        {"name": "ann", "age": 3, "tags": ["a"], "address": {"zip": "12345"}},
        {"name": "", "age": -17, "tags": ["a", "c d", "b"], "score": 1.5e3, "address": {"zip": "00000", "ok": True}, "nick": "x\"y"},
        {"name": "é\\n", "age": 0, "tags": ["b"], "score": None, "address": {"zip": "99999"}},
    ]
    for doc in good:
        assert _conforms(doc)
        assert dfa.fullmatch(json.dumps(doc, separators=(",", ":"), ensure_ascii=False)), doc
        assert dfa.fullmatch(json.dumps(doc, separators=(", ", ": "), ensure_ascii=False)), doc
    bad = [
        {"name": "toolongname", "age": 3, "tags": ["a"], "address": {"zip": "12345"}},
        {"name": "ann", "age": 3.5, "tags": ["a"], "address": {"zip": "12345"}},
        {"name": "ann", "age": 3, "tags": [], "address": {"zip": "12345"}},
        {"name": "ann", "age": 3, "tags": ["z"], "address": {"zip": "12345"}},
        {"name": "ann", "age": 3, "tags": ["a"], "address": {"zip": "1234"}},
        {"name": "ann", "age": 3, "tags": ["a"]},
        {"age": 3, "name": "ann", "tags": ["a"], "address": {"zip": "12345"}},     # members out of declaration order
    ]
    for doc in bad:
        assert not dfa.fullmatch(json.dumps(doc, separators=(",", ":"))), doc
    # random walks through the automaton always end in conforming JSON
    rng = random.Random(3)
    done = 0
    for _ in range(60):
        s, out = 0, bytearray()
        for _ in range(400):
            if dfa.accepting[s] and (not dfa.has_continuation(s) or rng.random() < 0.3):
                break
            nxt = [b for b in range(32, 127) if dfa.step(s, b) >= 0]
            if not nxt:
                break
            # steer towards closing brackets and quotes so that walks terminate
            pref = [b for b in nxt if chr(b) in '"}],:']
            b = rng.choice(pref) if pref and rng.random() < 0.5 else rng.choice(nxt)
            out.append(b)
            s = dfa.step(s, b)
        if dfa.accepting[s]:
            done += 1
            assert _conforms(json.loads(out.decode())), out
    assert done >= 10


def test_free_form_json_and_optional_members():
    anyj = DFA(json_schema_to_regex({}))
    for text in ['{"a": [1, 2, {"b": null}], "c": "x"}', "[]", "3.5e-2", '"s"', '{"k":{"k":[true]}}']:
        json.loads(text)
        assert anyj.fullmatch(text), text
    for text in ["{", '{"a":}', "[1,]", "tru", '{"k":{"k":{"k":{"k":{"k":1}}}}}']:      # the last one nests deeper than 3
        assert not anyj.fullmatch(text), text
    opt = DFA(json_schema_to_regex({"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "boolean"},
                                                                      "c": {"type": "null"}}, "required": ["b"]}))
    for text, want in [('{"b":true}', True), ('{"a":1,"b":false}', True), ('{"b":true,"c":null}', True),
                       ('{"a":1,"b":false,"c":null}', True), ('{"a":1}', False), ('{"b":true,}', False), ('{,"b":true}', False),
                       ('{"c":null,"b":true}', False)]:
        assert opt.fullmatch(text) == want, text


def test_token_masks_equal_brute_force():
    rng = random.Random(0)
    pieces = ['{"', '"', "}", "{", ":", ",", " ", "true", "false", "tr", "ue", "null", "nu", "ll", "a", "b", '":', '",', "12",
              "3", "-", ".", "e", '"}', "[", "]", '["', '"]', "é", "\\", "n", "0"]
    table = [b""] + [p.encode() for p in pieces] + [bytes([rng.randrange(97, 123) for _ in range(rng.randrange(1, 4))])
                                                    for _ in range(200)]
    eos = 0
    trie = TokenTrie(table)
    dfa = DFA(json_schema_to_regex({"type": "object", "properties": {"a": {"type": "boolean"}, "b": {"type": "string", "maxLength": 4}},
                                    "required": ["a", "b"]}))
    fsm = GuidedFSM(dfa, trie, eos)
    # drive generation by always picking a random allowed token; every prefix state's mask equals brute force
    for _ in range(40):
        hist = []
        for _ in range(60):
            s = fsm.state_after(hist)
            assert s >= 0
            allowed = fsm.allowed_tokens(s)
            brute = sorted([t for t, bs in enumerate(table) if bs and dfa.walk(bs, s) >= 0] + ([eos] if dfa.accepting[s] else []))
            assert allowed == brute
            assert allowed, "a live state always has a way on"
            t = rng.choice(allowed)
            if t == eos:
                break
            hist.append(t)
        text = b"".join(table[t] for t in hist).decode()
        if dfa.accepting[fsm.state_after(hist)]:
            v = json.loads(text)
            assert isinstance(v["a"], bool) and isinstance(v["b"], str)


def test_constrained_generation_end_to_end():
    """Random-weight model, byte tokenizer: sampled text must match the regex / satisfy the schema, requests with
    and without a constraint share a batch, and a bad pattern is refused at submission."""
    from tokenweave_b200 import LLM, SamplingParams
    llm = LLM("tiny-llama", dtype="float32", device="cpu", block_size=16, max_num_batched_tokens=256, seed=3)
    date = r"(19|20)\d{2}-(0[1-9]|1[0-2])-(0[1-9]|[12]\d|3[01])"
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"},
                                               "tag": {"enum": ["red", "green"]}}, "required": ["ok", "n", "tag"]}
    sps = [SamplingParams(temperature=1.0, seed=1, max_tokens=40, guided_regex=date),
           SamplingParams(temperature=0.0, max_tokens=12),
           SamplingParams(temperature=1.0, seed=2, max_tokens=120, guided_json=schema),
           SamplingParams(temperature=0.8, seed=5, max_tokens=200, guided_json={"type": "array", "items": {"type": "integer"},
                                                                                "maxItems": 4})]
    outs = llm.generate(["date: ", "free text", "json: ", "list: "], sps)
    assert re.fullmatch(date, outs[0].outputs[0].text), outs[0].outputs[0].text
    assert outs[0].outputs[0].finish_reason == "stop"
    assert len(outs[1].outputs[0].token_ids) == 12
    doc = json.loads(outs[2].outputs[0].text)
    assert isinstance(doc["ok"], bool) and isinstance(doc["n"], int) and doc["tag"] in ("red", "green")
    arr = json.loads(outs[3].outputs[0].text)
    assert isinstance(arr, list) and len(arr) <= 4 and all(isinstance(x, int) for x in arr)
    with pytest.raises((RegexError, ValueError)):
        llm.generate(["x"], SamplingParams(guided_regex="(unclosed"))
    llm.shutdown()


def test_server_response_format():
    pytest.importorskip("fastapi")
    pytest.importorskip("httpx")
    from starlette.testclient import TestClient
    from tokenweave_b200.config import EngineArgs
    from tokenweave_b200.engine.async_engine import AsyncLLMEngine
    from tokenweave_b200.entrypoints.api_server import build_app
    eng = AsyncLLMEngine.from_engine_args(EngineArgs(model="tiny-llama", dtype="float32", device="cpu", block_size=16,
                                                     max_num_batched_tokens=128, seed=1))
    try:
        with TestClient(build_app(eng, "tiny")) as c:
            schema = {"type": "object", "properties": {"a": {"type": "boolean"}}, "required": ["a"]}
            r = c.post("/v1/completions", json={"prompt": "x", "max_tokens": 60, "temperature": 1.0, "seed": 4,
                                                "response_format": {"type": "json_schema", "json_schema": {"schema": schema}}})
            assert r.status_code == 200, r.text
            assert isinstance(json.loads(r.json()["choices"][0]["text"])["a"], bool)
            r = c.post("/v1/completions", json={"prompt": "x", "max_tokens": 30, "temperature": 1.0, "seed": 4,
                                                "guided_regex": "[ab]{3,5}!"})
            assert re.fullmatch("[ab]{3,5}!", r.json()["choices"][0]["text"])
            assert c.post("/v1/completions", json={"prompt": "x", "guided_regex": "(bad"}).status_code == 400
    finally:
        eng.shutdown()


def test_token_bytes_of_common_vocabulary_spellings():
    from tokenweave_b200.engine.structured import token_bytes_table

    class Fake:
        def __init__(self, pieces, special=()):
            self.pieces, self.all_special_ids = pieces, list(special)

        def convert_ids_to_tokens(self, ids):
            return [self.pieces[i] if i < len(self.pieces) else None for i in ids]

    # byte-level BPE: "Ġ" is a space, "Ċ" a newline, "Ã©" the two bytes of "é"
    bpe = Fake(["Ġhello", "Ċ", "Ã©", "{\"", "<|eot|>"], special=[4])
    assert token_bytes_table(bpe, 6) == [b" hello", b"\n", "é".encode(), b'{"', b"", b""]
    # sentencepiece: word-boundary marker and byte fallback
    sp = Fake(["▁the", "<0x0A>", "ab", "▁", "</s>"], special=[4])
    assert token_bytes_table(sp, 5) == [b" the", b"\n", b"ab", b" ", b""]


def test_constrained_text_is_always_well_formed_utf8():
    rng = random.Random(5)
    for pattern in [r'"[^"\\]*"', r"a.{0,6}b", json_schema_to_regex({"type": "string", "maxLength": 5})]:
        dfa = DFA(pattern)
        accepted = 0
        for _ in range(300):
            s, out = 0, bytearray()
            for _ in range(40):
                if dfa.accepting[s] and rng.random() < 0.3:
                    break
                nxt = [b for b in range(256) if dfa.step(s, b) >= 0]
                if not nxt:
                    break
                high = [b for b in nxt if b >= 0x80]
                b = rng.choice(high) if high and rng.random() < 0.6 else rng.choice(nxt)
                out.append(b)
                s = dfa.step(s, b)
            if dfa.accepting[s]:
                accepted += 1
                out.decode("utf-8")                 # raises on half a character, overlong forms, surrogates
        assert accepted > 5
    assert DFA(r"[^a]").fullmatch("é") and DFA(r".").fullmatch("😀") and not DFA(r".").fullmatch(b"\xc3")


ARITH = '''
root   ::= expr
expr   ::= term (("+" | "-") term)*          # sums of terms
term   ::= number | "(" expr ")"
number ::= [1-9] [0-9]{0,2}
'''


def _parse_arith(text: str) -> int:
    """Recursive-descent recogniser of ARITH; returns the deepest parenthesis nesting, raises on a syntax error."""
    pos, deepest = 0, 0

    def expr(depth: int) -> None:
        nonlocal pos
        term(depth)
        while pos < len(text) and text[pos] in "+-":
            pos += 1
            term(depth)

    def term(depth: int) -> None:
        nonlocal pos, deepest
        if pos < len(text) and text[pos] == "(":
            pos += 1
            deepest = max(deepest, depth + 1)
            expr(depth + 1)
            assert pos < len(text) and text[pos] == ")", text
            pos += 1
        else:
            start = pos
            while pos < len(text) and text[pos].isdigit():
                pos += 1
            assert 1 <= pos - start <= 3 and text[start] != "0", text

    expr(0)
    assert pos == len(text), text
    return deepest


def test_grammar_lowering_accepts_the_bounded_language():
    from tokenweave_b200.engine.structured import GrammarError, grammar_to_regex
    d = DFA(grammar_to_regex(ARITH, max_depth=2))
    for good in ["7", "12+3", "(1+2)-3", "((4))", "1-(2+(3))+999"]:
        assert d.fullmatch(good.encode()), good
        assert _parse_arith(good) <= 2
    for bad in ["", "1+", "()", "01", "1234", "(((5)))", "a", "1 + 2"]:
        assert not d.fullmatch(bad.encode()), bad
    assert DFA(grammar_to_regex(ARITH, max_depth=3)).fullmatch(b"(((5)))")
    # Lark-style colons, single quotes, a start rule by name, comments, repetition bounds, negated classes
    lark = """start: item (',' item){0,2}
item: [a-c]+ | '"' [^"]* '"'   # words or quoted text
"""
    d2 = DFA(grammar_to_regex(lark))
    assert d2.fullmatch(b'ab,"x y",c') and not d2.fullmatch(b"a,b,c,a") and not d2.fullmatch(b"d")
    with pytest.raises(GrammarError):
        grammar_to_regex("root ::= missing")
    with pytest.raises(GrammarError):
        grammar_to_regex('root ::= "(" root ")"')          # no derivation ends within the bound
    with pytest.raises(GrammarError):
        grammar_to_regex('root ::= ("a"')


def test_grammar_constrained_generation_end_to_end():
    """Sampled text of a random-weight model must be a sentence of the grammar; the server takes the same field."""
    from tokenweave_b200 import LLM, SamplingParams
    llm = LLM("tiny-llama", dtype="float32", device="cpu", block_size=16, max_num_batched_tokens=256, seed=3)
    outs = llm.generate(["calc: "] * 3, [SamplingParams(temperature=1.0, seed=s, max_tokens=60, guided_grammar=ARITH)
                                        for s in (1, 2, 3)])
    for o in outs:
        text = o.outputs[0].text
        if o.outputs[0].finish_reason == "stop":
            assert _parse_arith(text) <= 3, text             # a complete sentence within the nesting bound
        else:                                                # cut by max_tokens: still a prefix of a sentence
            assert all(c in "0123456789+-()" for c in text), text
    assert any(o.outputs[0].finish_reason == "stop" for o in outs)
    with pytest.raises(ValueError):
        llm.generate(["x"], SamplingParams(guided_grammar="root ::= nowhere"))
    llm.shutdown()
