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
