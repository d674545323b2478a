"""Function calling for the chat endpoint: the OpenAI ``tools`` / ``tool_choice`` fields.

Counterpart of vllm/entrypoints/openai/serving_chat.py (tool handling) and the parsers under
vllm/entrypoints/openai/tool_parsers/:

* ``tool_choice`` naming a function, or ``"required"``: the call is *forced* — the generation is constrained by
  a JSON schema built from the tools' parameter schemas (``engine/structured.py``), so the arguments always
  parse, whatever the model;
* ``tool_choice="auto"`` (the default when tools are given): the model decides; its text is scanned for calls in
  the spellings model families use (``--tool-call-parser`` of the server picks one, ``auto`` tries them in turn):
  ``hermes`` ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` blocks (Hermes, Qwen2.5);
  ``llama3_json`` a bare JSON object, list of objects or ``;``-separated objects with ``name`` and ``arguments`` /
  ``parameters`` keys (Llama-3.x); ``mistral`` ``[TOOL_CALLS]`` followed by a JSON list; ``pythonic`` a Python list of
  calls, ``[get_weather(city="Paris"), f(x=1)]`` (Llama-3.2 / 4 pythonic style).

``split_reasoning`` is the reasoning parser (``--reasoning-parser deepseek_r1``): text inside ``<think> ... </think>``
goes to ``reasoning_content``, the rest stays the answer (vllm/reasoning/deepseek_r1_reasoning_parser.py).
"""
from __future__ import annotations

import ast
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


TOOL_CALL_PARSERS = ("auto", "hermes", "llama3_json", "mistral", "pythonic")


def _parse_hermes(text: str, known: set) -> tuple[str, list[dict]]:
    found, rest = [], text
    for m in _HERMES.finditer(text):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        if isinstance(obj, dict) and obj.get("name") in known:
            found.append(_call(obj["name"], obj.get("arguments", obj.get("parameters"))))
            rest = rest.replace(m.group(0), "")
    return rest, found


def _calls_of_json(obj, known: set) -> list[dict]:
    items = obj if isinstance(obj, list) else [obj]
    if items and all(isinstance(c, dict) and c.get("name") in known for c in items):
        return [_call(c["name"], c.get("arguments", c.get("parameters"))) for c in items]
    return []


def _parse_llama3_json(text: str, known: set) -> tuple[str, list[dict]]:
    stripped = text.strip()
    if stripped.startswith("<|python_tag|>"):
        stripped = stripped[len("<|python_tag|>"):].strip()
    if stripped[:1] not in "{[":
        return text, []
    try:
        found = _calls_of_json(json.loads(stripped), known)
    except json.JSONDecodeError:
        found = []
        parts = [p.strip() for p in stripped.split(";") if p.strip()]       # several objects separated by ';'
        try:
            objs = [json.loads(p) for p in parts]
        except json.JSONDecodeError:
            objs = []
        if len(objs) > 1:
            found = _calls_of_json(objs, known)
    return ("" if found else text), found


def _parse_mistral(text: str, known: set) -> tuple[str, list[dict]]:
    tag = "[TOOL_CALLS]"
    at = text.find(tag)
    if at < 0:
        return text, []
    body = text[at + len(tag):].strip()
    try:
        obj, end = json.JSONDecoder().raw_decode(body)
    except json.JSONDecodeError:
        return text, []
    found = _calls_of_json(obj, known)
    return ((text[:at] + body[end:]) if found else text), found


def _parse_pythonic(text: str, known: set) -> tuple[str, list[dict]]:
    stripped = text.strip()
    if not (stripped.startswith("[") and stripped.endswith("]")):
        return text, []
    try:
        tree = ast.parse(stripped, mode="eval")
    except SyntaxError:
        return text, []
    if not isinstance(tree.body, ast.List) or not tree.body.elts:
        return text, []
    found = []
    for node in tree.body.elts:
        if not (isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id in known
                and not node.args):
            return text, []
        try:
            args = {kw.arg: ast.literal_eval(kw.value) for kw in node.keywords if kw.arg is not None}
        except (ValueError, SyntaxError):
            return text, []                 # an argument that is not a literal: leave the text alone
        found.append(_call(node.func.id, args))
    return "", found


_PARSERS = {"hermes": _parse_hermes, "llama3_json": _parse_llama3_json, "mistral": _parse_mistral,
            "pythonic": _parse_pythonic}


def calls_from_text(text: str, tools: list, parser: str = "auto") -> tuple[Optional[str], list[dict]]:
    """(remaining content, tool calls) found in free text; calls to unknown functions are left as text. ``parser``
    names the spelling to look for (see the module text); ``auto`` tries every one and takes the first that finds
    calls."""
    if parser not in TOOL_CALL_PARSERS:
        raise ValueError(f"unknown tool-call parser {parser!r} (one of {', '.join(TOOL_CALL_PARSERS)})")
    known = {f["name"] for f in _functions(tools)}
    order = list(_PARSERS) if parser == "auto" else [parser]
    for name in order:
        rest, found = _PARSERS[name](text, known)
        if found:
            rest = rest.strip()
            return (rest or None), found
    return text, []


_THINK = re.compile(r"<think>(.*?)</think>", re.S)


def split_reasoning(text: str) -> tuple[Optional[str], Optional[str]]:
    """(reasoning, answer) of a completion that wraps its reasoning in ``<think> ... </think>``. A completion that
    only closes the block (the template opened it) counts everything before ``</think>`` as reasoning; one that
    never closes it is all reasoning (it was cut off before the answer)."""
    m = _THINK.search(text)
    if m:
        answer = (text[:m.start()] + text[m.end():]).strip()
        return m.group(1).strip() or None, answer or None
    if "</think>" in text:
        head, tail = text.split("</think>", 1)
        return head.replace("<think>", "").strip() or None, tail.strip() or None
    if "<think>" in text:
        return text.split("<think>", 1)[1].strip() or None, None
    return None, text


def describe_tools(tools: list) -> str:
    """Plain-text description for prompts of tokenizers without a tool-aware chat template."""
    lines = ["You may call these functions by answering with "
             '<tool_call>{"name": <function name>, "arguments": <JSON object>}</tool_call>:']
    for f in _functions(tools):
        lines.append(json.dumps({"name": f["name"], "description": f.get("description", ""),
                                 "parameters": f.get("parameters", {})}))
    return "\n".join(lines)
