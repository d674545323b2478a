"""Function calling for the chat endpoint: the OpenAI ``tools`` / ``tool_choice`` fields.

Counterpart of vllm/entrypoints/openai/serving_chat.py (tool handling) and the parsers under
vllm/entrypoints/openai/tool_parsers/:

* ``tool_choice`` naming a function, or ``"required"``: the call is *forced* — the generation is constrained by
  a JSON schema built from the tools' parameter schemas (``engine/structured.py``), so the arguments always
  parse, whatever the model;
* ``tool_choice="auto"`` (the default when tools are given): the model decides; its text is scanned for calls in
  the two common spellings, Hermes-style ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` blocks and a
  bare JSON object (or list of objects) with ``name`` and ``arguments`` / ``parameters`` keys (Llama-3 JSON style).
"""
from __future__ import annotations

import json
import re
import uuid
from typing import Any, Optional


def _functions(tools: list) -> list[dict]:
    out = []
    for t in tools or []:
        f = t.get("function", t) if isinstance(t, dict) else None
        if not isinstance(f, dict) or "name" not in f:
            raise ValueError("every tool needs a function with a name")
        out.append(f)
    return out


def forced_schema(tools: list, tool_choice: Any) -> Optional[dict]:
    """JSON schema the output must satisfy when a call is forced; None when the model is free to answer in text.
    A named function yields the schema of its arguments; ``"required"`` a one-element list of calls."""
    if tool_choice in (None, "auto", "none") or not tools:
        return None
    funcs = _functions(tools)
    if isinstance(tool_choice, dict):
        name = (tool_choice.get("function") or {}).get("name", tool_choice.get("name"))
        for f in funcs:
            if f["name"] == name:
                return f.get("parameters") or {"type": "object", "properties": {}}
        raise ValueError(f"tool_choice names {name!r}, which is not among the tools")
    if tool_choice == "required":
        calls = [{"type": "object", "properties": {"name": {"const": f["name"]},
                                                   "parameters": f.get("parameters") or {"type": "object", "properties": {}}},
                  "required": ["name", "parameters"]} for f in funcs]
        return {"type": "array", "minItems": 1, "maxItems": 1, "items": {"anyOf": calls}}
    raise ValueError(f"unsupported tool_choice {tool_choice!r}")


def _call(name: str, arguments: Any) -> dict:
    args = arguments if isinstance(arguments, str) else json.dumps(arguments if arguments is not None else {})
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function", "function": {"name": name, "arguments": args}}


def calls_from_forced(text: str, tools: list, tool_choice: Any) -> list[dict]:
    """Tool calls of a generation that ran under :func:`forced_schema`."""
    data = json.loads(text)
    if isinstance(tool_choice, dict):
        name = (tool_choice.get("function") or {}).get("name", tool_choice.get("name"))
        return [_call(name, data)]
    return [_call(c["name"], c.get("parameters", {})) for c in data]


_HERMES = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.DOTALL)


def calls_from_text(text: str, tools: list) -> tuple[Optional[str], list[dict]]:
    """(remaining content, tool calls) found in free text; calls to unknown functions are left as text."""
    known = {f["name"] for f in _functions(tools)}
    found, rest = [], text
    for m in _HERMES.finditer(text):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        if isinstance(obj, dict) and obj.get("name") in known:
            found.append(_call(obj["name"], obj.get("arguments", obj.get("parameters"))))
            rest = rest.replace(m.group(0), "")
    if not found:
        stripped = text.strip()
        if stripped[:1] in "{[":
            try:
                obj = json.loads(stripped)
            except json.JSONDecodeError:
                obj = None
            items = obj if isinstance(obj, list) else [obj]
            if items and all(isinstance(c, dict) and c.get("name") in known for c in items):
                found = [_call(c["name"], c.get("arguments", c.get("parameters"))) for c in items]
                rest = ""
    rest = rest.strip()
    return (rest or None) if found else text, found


def describe_tools(tools: list) -> str:
    """Plain-text description for prompts of tokenizers without a tool-aware chat template."""
    lines = ["You may call these functions by answering with "
             '<tool_call>{"name": <function name>, "arguments": <JSON object>}</tool_call>:']
    for f in _functions(tools):
        lines.append(json.dumps({"name": f["name"], "description": f.get("description", ""),
                                 "parameters": f.get("parameters", {})}))
    return "\n".join(lines)
