"""Function calling in the chat endpoint: forced calls run under a JSON-schema constraint, free text is scanned
for Hermes-style and bare-JSON calls."""
import json

import pytest

from tokenweave_b200.entrypoints import tool_calls as tc

TOOLS = [
    {"type": "function", "function": {"name": "get_weather", "description": "weather of a city",
                                      "parameters": {"type": "object", "properties": {
                                          "city": {"type": "string", "maxLength": 8},
                                          "unit": {"enum": ["c", "f"]}}, "required": ["city", "unit"]}}},
    {"type": "function", "function": {"name": "add", "parameters": {"type": "object", "properties": {
        "a": {"type": "integer"}, "b": {"type": "integer"}}, "required": ["a", "b"]}}},
]


def test_parsers_and_schemas():
    assert tc.forced_schema(TOOLS, "auto") is None and tc.forced_schema(TOOLS, None) is None
    named = tc.forced_schema(TOOLS, {"type": "function", "function": {"name": "add"}})
    assert named["required"] == ["a", "b"]
    with pytest.raises(ValueError):
        tc.forced_schema(TOOLS, {"type": "function", "function": {"name": "nope"}})
    content, calls = tc.calls_from_text('ok <tool_call>{"name": "add", "arguments": {"a": 1, "b": 2}}</tool_call>', TOOLS)
    assert content == "ok" and calls[0]["function"] == {"name": "add", "arguments": '{"a": 1, "b": 2}'}
    content, calls = tc.calls_from_text('[{"name": "get_weather", "parameters": {"city": "Oslo", "unit": "c"}}]', TOOLS)
    assert content is None and json.loads(calls[0]["function"]["arguments"]) == {"city": "Oslo", "unit": "c"}
    content, calls = tc.calls_from_text('{"name": "unknown", "arguments": {}}', TOOLS)       # not one of ours: text
    assert calls == [] and content.startswith("{")
    assert tc.calls_from_text("just words", TOOLS) == ("just words", [])


def test_chat_endpoint_with_tools():
    pytest.importorskip("fastapi")
    pytest.importorskip("httpx")
    from starlette.testclient import TestClient
    from tokenweave_b200.config import EngineArgs
    from tokenweave_b200.engine.async_engine import AsyncLLMEngine
    from tokenweave_b200.entrypoints.api_server import build_app
    eng = AsyncLLMEngine.from_engine_args(EngineArgs(model="tiny-llama", dtype="float32", device="cpu", block_size=16,
                                                     max_num_batched_tokens=512, seed=1))
    msgs = [{"role": "user", "content": "weather in Oslo?"}]
    try:
        with TestClient(build_app(eng, "tiny")) as c:
            body = {"messages": msgs, "tools": TOOLS, "max_tokens": 200, "temperature": 1.0, "seed": 3}
            # a named function: the arguments satisfy its schema whatever the (random) model would like to say
            r = c.post("/v1/chat/completions", json={**body, "tool_choice": {"type": "function",
                                                                              "function": {"name": "get_weather"}}})
            assert r.status_code == 200, r.text
            ch = r.json()["choices"][0]
            assert ch["finish_reason"] == "tool_calls" and ch["message"]["content"] is None
            call = ch["message"]["tool_calls"][0]
            args = json.loads(call["function"]["arguments"])
            assert call["function"]["name"] == "get_weather" and args["unit"] in ("c", "f") and len(args["city"]) <= 8
            # "required": some function of the list, with arguments of that function's schema
            r = c.post("/v1/chat/completions", json={**body, "tool_choice": "required", "seed": 5})
            call = r.json()["choices"][0]["message"]["tool_calls"][0]
            args = json.loads(call["function"]["arguments"])
            want = {"add": {"a", "b"}, "get_weather": {"city", "unit"}}
            assert set(args) == want[call["function"]["name"]]
            # "auto" with a model that produces no call: plain content, and tool_choice "none" ignores the tools
            r = c.post("/v1/chat/completions", json={**body, "max_tokens": 8, "temperature": 0})
            assert "tool_calls" not in r.json()["choices"][0]["message"]
            r = c.post("/v1/chat/completions", json={**body, "tool_choice": "none", "max_tokens": 4})
            assert r.json()["choices"][0]["message"]["content"] is not None
            # streaming with tools: one chunk carrying the whole message
            chunks = []
            with c.stream("POST", "/v1/chat/completions",
                          json={**body, "stream": True, "tool_choice": {"type": "function", "function": {"name": "add"}}}) as s:
                for line in s.iter_lines():
                    if line.startswith("data: ") and line != "data: [DONE]":
                        chunks.append(json.loads(line[6:]))
            delta = chunks[0]["choices"][0]["delta"]
            assert set(json.loads(delta["tool_calls"][0]["function"]["arguments"])) == {"a", "b"}
            assert c.post("/v1/chat/completions", json={**body, "tool_choice": {"function": {"name": "zzz"}}}).status_code == 400
    finally:
        eng.shutdown()


def test_named_parsers_and_reasoning_split():
    """The spellings of the model families, each alone and through ``auto``; the <think> splitter."""
    mistral = '[TOOL_CALLS] [{"name": "get_weather", "arguments": {"city": "Paris", "unit": "c"}}]'
    pythonic = '[get_weather(city="Paris", unit="c"), add(a=1, b=2)]'
    semis = '{"name": "add", "parameters": {"a": 1, "b": 2}}; {"name": "add", "parameters": {"a": 3, "b": 4}}'
    hermes = 'sure <tool_call>{"name": "add", "arguments": {"a": 1, "b": 2}}</tool_call>'
    for text, parser, n in ((mistral, "mistral", 1), (pythonic, "pythonic", 2), (semis, "llama3_json", 2),
                            (hermes, "hermes", 1)):
        for p in (parser, "auto"):
            content, calls = tc.calls_from_text(text, TOOLS, p)
            assert len(calls) == n and all(c["type"] == "function" for c in calls), (p, text)
        # another family's parser leaves the text alone
        other = "hermes" if parser != "hermes" else "mistral"
        assert tc.calls_from_text(text, TOOLS, other) == (text, [])
    _, calls = tc.calls_from_text(pythonic, TOOLS, "pythonic")
    assert json.loads(calls[1]["function"]["arguments"]) == {"a": 1, "b": 2}
    # not calls: an unknown function, positional arguments, a non-literal argument, a plain list
    for text in ('[nope(a=1)]', '[add(1, 2)]', '[add(a=x, b=2)]', '[1, 2]'):
        assert tc.calls_from_text(text, TOOLS, "pythonic") == (text, [])
    with pytest.raises(ValueError):
        tc.calls_from_text("x", TOOLS, "xml")
    assert tc.split_reasoning("<think>two plus two</think> 4") == ("two plus two", "4")
    assert tc.split_reasoning("carry the one</think>12") == ("carry the one", "12")
    assert tc.split_reasoning("<think>never finished") == ("never finished", None)
    assert tc.split_reasoning("no tags") == (None, "no tags")


def test_server_options_for_parsers():
    pytest.importorskip("fastapi")
    from tokenweave_b200.config import EngineArgs
    from tokenweave_b200.engine.async_engine import AsyncLLMEngine
    from tokenweave_b200.entrypoints.api_server import build_app
    pytest.importorskip("httpx")
    from starlette.testclient import TestClient
    eng = AsyncLLMEngine.from_engine_args(EngineArgs(model="tiny-llama", dtype="float32", device="cpu", block_size=16,
                                                     max_num_batched_tokens=256, seed=1))
    try:
        with pytest.raises(ValueError):
            build_app(eng, "tiny", tool_call_parser="xml")
        with pytest.raises(ValueError):
            build_app(eng, "tiny", reasoning_parser="other")
        with TestClient(build_app(eng, "tiny", tool_call_parser="pythonic", reasoning_parser="deepseek_r1")) as c:
            r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6,
                                                     "temperature": 0})
            msg = r.json()["choices"][0]["message"]
            assert r.status_code == 200 and msg["content"] is not None and "reasoning_content" not in msg
    finally:
        eng.shutdown()
