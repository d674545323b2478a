"""Structured output: generation constrained to a regular expression or a JSON schema.

The reference delegates this to external grammar engines (xgrammar / guidance behind
vllm/v1/structured_output/, requested through ``GuidedDecodingParams`` in vllm/sampling_params.py) and applies
the resulting token bitmask to the logits before sampling. Neither engine is available here, so the same
contract is implemented directly:

* a regular expression (the ``re`` subset below) is parsed and compiled to a byte-level NFA, determinised
  lazily;
* a JSON schema is lowered to such an expression (``json_schema_to_regex``; recursion and free-form values are
  expanded to a bounded nesting depth, which keeps the language regular);
* the tokenizer's vocabulary is arranged in a byte trie once; for a DFA state the allowed tokens are found by
  walking trie and DFA together, which prunes a token at its first impossible byte. Masks are cached per state.

The sampler asks :class:`GuidedFSM` for the mask of the state reached by the tokens generated so far; the
end-of-sequence token is allowed exactly in accepting states, which is also how generation terminates.

Supported syntax: literals, ``.``, escapes ``\\d \\w \\s \\D \\W \\S \\n \\t \\r \\xHH \\uHHHH`` and escaped
punctuation, classes ``[a-z0-9_]`` / ``[^...]``, groups ``( )`` and ``(?: )``, alternation, ``* + ?`` and
``{m} {m,} {m,n}`` (a lazy ``?`` suffix is accepted and ignored; ``^`` / ``$`` at the ends are ignored since
the whole output must match). ``\\d \\w \\s`` are the ASCII classes. Characters outside ASCII are matched as their
UTF-8 byte sequences; ``.`` and negated classes accept any whole, well-formed multi-byte character, so a
constrained output is always valid UTF-8.
"""
from __future__ import annotations

import json
from collections import OrderedDict
from typing import Optional, Sequence, Union

ALL = (1 << 256) - 1
_HIGH = sum(1 << b for b in range(0x80, 0x100))


def _mask(chars) -> int:
    m = 0
    for c in chars:
        m |= 1 << (c if isinstance(c, int) else ord(c))
    return m


_DIGIT = _mask("0123456789")
_WORD = _DIGIT | _mask("abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ_")
_SPACE = _mask(" \t\n\r\f\v")
_ASCII = (1 << 128) - 1
_CLASS_ESC = {"d": _DIGIT, "w": _WORD, "s": _SPACE, "D": (ALL & ~_DIGIT), "W": (ALL & ~_WORD), "S": (ALL & ~_SPACE)}
_CHAR_ESC = {"n": "\n", "t": "\t", "r": "\r", "f": "\f", "v": "\v", "0": "\0", "a": "\a", "b": "\b"}


class RegexError(ValueError):
    pass


def _range_mask(lo: int, hi: int) -> int:
    return sum(1 << b for b in range(lo, hi + 1))


def _utf8_multibyte():
    """AST of one well-formed multi-byte UTF-8 character (no overlong forms, no surrogates, up to U+10FFFF), so
    that ``.`` and negated classes never let half a character through."""
    tail = ("set", _range_mask(0x80, 0xBF))
    seq = lambda *parts: ("cat", [p if isinstance(p, tuple) else ("set", p) for p in parts])  # noqa: E731
    return ("alt", [
        seq(_range_mask(0xC2, 0xDF), tail),
        seq(1 << 0xE0, _range_mask(0xA0, 0xBF), tail),
        seq(_range_mask(0xE1, 0xEC) | _range_mask(0xEE, 0xEF), tail, tail),
        seq(1 << 0xED, _range_mask(0x80, 0x9F), tail),
        seq(1 << 0xF0, _range_mask(0x90, 0xBF), tail, tail),
        seq(_range_mask(0xF1, 0xF3), tail, tail, tail),
        seq(1 << 0xF4, _range_mask(0x80, 0x8F), tail, tail),
    ])


# ---- parser: pattern -> AST ------------------------------------------------------------------------------------
# AST: ("set", mask) | ("cat", [nodes]) | ("alt", [nodes]) | ("rep", node, lo, hi or None)
class _Parser:
    def __init__(self, pattern: str):
        self.p = pattern
        self.i = 0

    def parse(self):
        if self.p.startswith("^"):
            self.i = 1
        node = self._alt()
        if self.i < len(self.p):
            raise RegexError(f"unexpected {self.p[self.i]!r} at {self.i} in {self.p!r}")
        return node

    def _peek(self) -> Optional[str]:
        return self.p[self.i] if self.i < len(self.p) else None

    def _alt(self):
        branches = [self._cat()]
        while self._peek() == "|":
            self.i += 1
            branches.append(self._cat())
        return branches[0] if len(branches) == 1 else ("alt", branches)

    def _cat(self):
        items = []
        while self._peek() is not None and self._peek() not in "|)":
            if self._peek() == "$" and self.i == len(self.p) - 1:
                self.i += 1
                break
            items.append(self._repeat())
        return ("cat", items)

    def _repeat(self):
        node = self._atom()
        while True:
            c = self._peek()
            if c == "*":
                lo, hi = 0, None
            elif c == "+":
                lo, hi = 1, None
            elif c == "?":
                lo, hi = 0, 1
            elif c == "{":
                j = self.p.find("}", self.i)
                body = self.p[self.i + 1:j] if j > 0 else ""
                parts = body.split(",")
                if j < 0 or not all(x.strip().isdigit() or x.strip() == "" for x in parts) or len(parts) > 2 or not parts[0].strip():
                    raise RegexError(f"bad quantifier at {self.i} in {self.p!r}")
                lo = int(parts[0])
                hi = lo if len(parts) == 1 else (int(parts[1]) if parts[1].strip() else None)
                if hi is not None and hi < lo:
                    raise RegexError("quantifier bounds out of order")
                self.i = j
            else:
                return node
            self.i += 1
            if self._peek() == "?":         # lazy variants match the same language
                self.i += 1
            node = ("rep", node, lo, hi)

    def _escape(self, in_class: bool):
        """After a backslash: returns a mask (class escape) or a character."""
        c = self._peek()
        if c is None:
            raise RegexError("dangling backslash")
        self.i += 1
        if c in _CLASS_ESC:
            return _CLASS_ESC[c]
        if c == "x":
            h = self.p[self.i:self.i + 2]
            self.i += 2
            return chr(int(h, 16))
        if c == "u":
            h = self.p[self.i:self.i + 4]
            self.i += 4
            return chr(int(h, 16))
        if c == "b" and not in_class:
            raise RegexError("word boundaries are not supported")
        if c in _CHAR_ESC:
            return _CHAR_ESC[c]
        if c.isalnum():
            raise RegexError(f"unsupported escape \\{c}")
        return c

    @staticmethod
    def _literal(ch: str):
        bs = ch.encode("utf-8")
        if len(bs) == 1:
            return ("set", 1 << bs[0])
        return ("cat", [("set", 1 << b) for b in bs])

    def _atom(self):
        c = self._peek()
        self.i += 1
        if c == "(":
            if self.p.startswith("?:", self.i):
                self.i += 2
            elif self._peek() == "?":
                raise RegexError("look-around and named groups are not supported")
            node = self._alt()
            if self._peek() != ")":
                raise RegexError(f"missing ) in {self.p!r}")
            self.i += 1
            return node
        if c == "[":
            return self._class()
        if c == ".":
            return ("alt", [("set", _ASCII & ~(1 << 0x0A)), _utf8_multibyte()])
        if c == "\\":
            e = self._escape(False)
            return ("set", e) if isinstance(e, int) else self._literal(e)
        if c in "*+?{":
            raise RegexError(f"nothing to repeat at {self.i - 1} in {self.p!r}")
        return self._literal(c)

    def _class(self):
        negate = self._peek() == "^"
        if negate:
            self.i += 1
        mask, wide = 0, []              # wide: non-ASCII members, matched as byte sequences
        first = True
        while True:
            c = self._peek()
            if c is None:
                raise RegexError(f"missing ] in {self.p!r}")
            if c == "]" and not first:
                self.i += 1
                break
            first = False
            self.i += 1
            lo = self._escape(True) if c == "\\" else c
            if isinstance(lo, int):
                mask |= lo
                continue
            if self._peek() == "-" and self.i + 1 < len(self.p) and self.p[self.i + 1] != "]":
                self.i += 1
                h = self._peek()
                self.i += 1
                hi = self._escape(True) if h == "\\" else h
                if isinstance(hi, int) or ord(hi) < ord(lo):
                    raise RegexError("bad character range")
                for o in range(ord(lo), ord(hi) + 1):
                    if o < 128:
                        mask |= 1 << o
                    elif o - ord(lo) < 4096:
                        wide.append(chr(o))
                    else:
                        raise RegexError("character range too wide")
            elif ord(lo) < 128:
                mask |= 1 << ord(lo)
            else:
                wide.append(lo)
        if negate:
            # complement over ASCII, plus any whole multi-byte character (non-ASCII members are not excluded)
            return ("alt", [("set", _ASCII & ~mask), _utf8_multibyte()])
        if not wide:
            return ("set", mask)
        return ("alt", ([("set", mask)] if mask else []) + [self._literal(ch) for ch in wide])


# ---- AST -> NFA --------------------------------------------------------------------------------------------------
class _NFA:
    def __init__(self):
        self.eps: list[list[int]] = []
        self.edges: list[list[tuple[int, int]]] = []      # state -> [(byte mask, target)]

    def new(self) -> int:
        self.eps.append([])
        self.edges.append([])
        return len(self.eps) - 1

    def build(self, node, start: int) -> int:
        """Attach ``node`` behind ``start``; returns its end state."""
        kind = node[0]
        if kind == "set":
            end = self.new()
            self.edges[start].append((node[1], end))
            return end
        if kind == "cat":
            cur = start
            for n in node[1]:
                cur = self.build(n, cur)
            return cur
        if kind == "alt":
            end = self.new()
            for n in node[1]:
                s = self.new()
                self.eps[start].append(s)
                self.eps[self.build(n, s)].append(end)
            return end
        _, sub, lo, hi = node
        if len(self.eps) > 400_000:
            raise RegexError("expression too large")
        cur = start
        for _ in range(lo):
            cur = self.build(sub, cur)
        if hi is None:
            loop = self.new()
            self.eps[cur].append(loop)
            self.eps[self.build(sub, loop)].append(loop)
            return loop
        end = self.new()
        self.eps[cur].append(end)
        for _ in range(hi - lo):
            cur = self.build(sub, cur)
            self.eps[cur].append(end)
        return end


class DFA:
    """Lazily determinised automaton over bytes. State 0 is the start; ``step`` returns -1 for a dead end."""

    def __init__(self, pattern: str):
        self.pattern = pattern
        nfa = _NFA()
        start = nfa.new()
        self._accept_nfa = nfa.build(_Parser(pattern).parse(), start)
        self._nfa = nfa
        self._ids: dict[frozenset, int] = {}
        self._sets: list[frozenset] = []
        self._trans: list[dict[int, int]] = []
        self.accepting: list[bool] = []
        self._intern(self._closure({start}))

    def _closure(self, states) -> frozenset:
        stack, seen = list(states), set(states)
        while stack:
            for t in self._nfa.eps[stack.pop()]:
                if t not in seen:
                    seen.add(t)
                    stack.append(t)
        return frozenset(seen)

    def _intern(self, fs: frozenset) -> int:
        i = self._ids.get(fs)
        if i is None:
            i = len(self._sets)
            self._ids[fs] = i
            self._sets.append(fs)
            self._trans.append({})
            self.accepting.append(self._accept_nfa in fs)
        return i

    def step(self, state: int, byte: int) -> int:
        t = self._trans[state]
        n = t.get(byte)
        if n is None:
            bit = 1 << byte
            targets = {to for s in self._sets[state] for m, to in self._nfa.edges[s] if m & bit}
            n = self._intern(self._closure(targets)) if targets else -1
            t[byte] = n
        return n

    def walk(self, data: bytes, state: int = 0) -> int:
        for b in data:
            state = self.step(state, b)
            if state < 0:
                return -1
        return state

    def fullmatch(self, text: Union[str, bytes]) -> bool:
        s = self.walk(text.encode("utf-8") if isinstance(text, str) else text)
        return s >= 0 and self.accepting[s]

    def has_continuation(self, state: int) -> bool:
        """True if some byte leads on from ``state`` (the output may still grow)."""
        return any(m for s in self._sets[state] for m, _ in self._nfa.edges[s])


# ---- JSON schema -> regex ------------------------------------------------------------------------------------
_WS = "[ ]?"
_STR_CHAR = r'([^"\\\x00-\x1f]|\\["\\/bfnrt]|\\u[0-9a-fA-F]{4})'
_INT = r"-?(0|[1-9][0-9]*)"
_NUM = _INT + r"(\.[0-9]+)?([eE][+-]?[0-9]+)?"
_SPECIAL = set(".^$*+?{}[]\\|()")


def regex_escape(text: str) -> str:
    return "".join("\\" + c if c in _SPECIAL else ("\\n" if c == "\n" else c) for c in text)


def _any_json(depth: int) -> str:
    scalar = f'"{_STR_CHAR}*"|{_NUM}|true|false|null'
    if depth <= 0:
        return f"({scalar})"
    inner = _any_json(depth - 1)
    arr = rf"\[{_WS}({inner}({_WS},{_WS}{inner})*)?{_WS}\]"
    member = f'"{_STR_CHAR}*"{_WS}:{_WS}{inner}'
    obj = rf"\{{{_WS}({member}({_WS},{_WS}{member})*)?{_WS}\}}"
    return f"({scalar}|{arr}|{obj})"


def json_schema_to_regex(schema: Union[str, dict, bool, None], max_depth: int = 3) -> str:
    """Regular expression of the JSON texts that satisfy ``schema`` (compact form, at most one space after
    separators). Supported keywords: type (also a list of types), enum, const, properties / required (members in
    declaration order, nothing additional), items / minItems / maxItems, minLength / maxLength / pattern,
    anyOf / oneOf, ``$ref`` into ``$defs`` / ``definitions``. A schema without a type (or ``True`` / ``{}``)
    admits any JSON value nested at most ``max_depth`` deep; recursive references are cut at the same depth."""
    if isinstance(schema, str):
        schema = json.loads(schema)
    root = schema if isinstance(schema, dict) else {}

    def resolve(ref: str) -> dict:
        if not ref.startswith("#/"):
            raise ValueError(f"only local $ref is supported, got {ref!r}")
        node = root
        for part in ref[2:].split("/"):
            node = node[part]
        return node

    def conv(s, depth: int) -> str:
        if s is True or s is None or s == {}:
            return _any_json(max(depth, 0))
        if s is False:
            raise ValueError("a false schema admits nothing")
        if "$ref" in s:
            if depth <= 0:
                raise ValueError("schema recursion deeper than max_depth")
            return conv(resolve(s["$ref"]), depth - 1)
        if "const" in s:
            return regex_escape(json.dumps(s["const"], separators=(",", ":"), ensure_ascii=False))
        if "enum" in s:
            return "(" + "|".join(regex_escape(json.dumps(v, separators=(",", ":"), ensure_ascii=False)) for v in s["enum"]) + ")"
        for key in ("anyOf", "oneOf"):
            if key in s:
                return "(" + "|".join(conv(x, depth) for x in s[key]) + ")"
        if "allOf" in s:
            if len(s["allOf"]) == 1:
                return conv(s["allOf"][0], depth)
            raise ValueError("allOf with several members is not supported")
        t = s.get("type")
        if isinstance(t, list):
            return "(" + "|".join(conv({**s, "type": x}, depth) for x in t) + ")"
        if t is None:
            t = "object" if "properties" in s else "array" if "items" in s else None
        if t is None:
            return _any_json(max(depth, 0))
        if t == "string":
            if "pattern" in s:
                return '"' + s["pattern"].lstrip("^").rstrip("$") + '"'
            lo, hi = s.get("minLength", 0), s.get("maxLength")
            q = "*" if (lo == 0 and hi is None) else f"{{{lo},{'' if hi is None else hi}}}"
            return f'"{_STR_CHAR}{q}"'
        if t == "integer":
            return _INT
        if t == "number":
            return _NUM
        if t == "boolean":
            return "(true|false)"
        if t == "null":
            return "null"
        if t == "array":
            item = conv(s.get("items", True), depth - 1)
            lo, hi = s.get("minItems", 0), s.get("maxItems")
            if hi is not None and hi == 0:
                return rf"\[{_WS}\]"
            more = f"({_WS},{_WS}{item})"
            tail = more + (f"{{{max(lo - 1, 0)},{'' if hi is None else hi - 1}}}")
            body = f"{item}{tail}"
            return rf"\[{_WS}{body}{_WS}\]" if lo > 0 else rf"\[{_WS}({body})?{_WS}\]"
        if t == "object":
            props = list(s.get("properties", {}).items())
            if not props:
                if s.get("additionalProperties", True) is False:
                    return rf"\{{{_WS}\}}"
                inner = conv(s["additionalProperties"], depth - 1) if isinstance(s.get("additionalProperties"), dict) \
                    else _any_json(max(depth - 1, 0))
                member = f'"{_STR_CHAR}*"{_WS}:{_WS}{inner}'
                return rf"\{{{_WS}({member}({_WS},{_WS}{member})*)?{_WS}\}}"
            required = set(s.get("required", []))
            members = [(f'"{regex_escape(json.dumps(name, ensure_ascii=False)[1:-1])}"{_WS}:{_WS}{conv(sub, depth - 1)}',
                        name in required) for name, sub in props]
            sep = f"{_WS},{_WS}"

            def rest(i: int) -> str:          # members i.. when at least one member precedes them
                return "".join(f"{sep}{m}" if req else f"({sep}{m})?" for m, req in members[i:])

            def lead(i: int) -> str:          # members i.. when nothing precedes them
                if i == len(members):
                    return ""
                m, req = members[i]
                if req:
                    return m + rest(i + 1)
                return f"({m}{rest(i + 1)}|{lead(i + 1)})"
            return rf"\{{{_WS}{lead(0)}{_WS}\}}"
        raise ValueError(f"unsupported schema type {t!r}")

    return conv(schema, max_depth)


# ---- vocabulary trie and token masks ---------------------------------------------------------------------------
# ---- context-free grammars, lowered to a regular expression of bounded nesting ----------------------------------
class GrammarError(ValueError):
    pass


class _GrammarParser:
    """GBNF / EBNF text -> ``{rule: alternatives}`` where an alternative is a list of items and an item is
    ``("lit", text)``, ``("class", source)``, ``("any",)``, ``("ref", name)``, ``("group", alternatives)`` or
    ``("rep", item, lo, hi)``. Rules are ``name ::= ...`` (``name: ...`` is accepted too), alternatives are
    separated by ``|``, items are string literals in double or single quotes, character classes ``[...]``, ``.``,
    rule names, parenthesised groups, each with an optional ``?`` ``*`` ``+`` or ``{m,n}``; ``#`` starts a comment.
    A rule ends where the next ``name ::=`` begins."""

    def __init__(self, text: str):
        self.t = text
        self.i = 0

    def _ws(self, newlines: bool = True) -> None:
        while self.i < len(self.t):
            c = self.t[self.i]
            if c == "#":
                while self.i < len(self.t) and self.t[self.i] != "\n":
                    self.i += 1
            elif c in " \t\r" or (newlines and c == "\n"):
                self.i += 1
            else:
                return

    def _name(self) -> Optional[str]:
        j = self.i
        while j < len(self.t) and (self.t[j].isalnum() or self.t[j] in "_-"):
            j += 1
        if j == self.i:
            return None
        name, self.i = self.t[self.i:j], j
        return name

    def _at_rule_start(self) -> bool:
        save = self.i
        name = self._name()
        ok = False
        if name is not None:
            self._ws(False)
            ok = self.t.startswith("::=", self.i) or (self.t.startswith(":", self.i) and not self.t.startswith("::", self.i))
        self.i = save
        return ok

    def parse(self) -> dict:
        rules: dict = {}
        self._ws()
        while self.i < len(self.t):
            name = self._name()
            if name is None:
                raise GrammarError(f"rule name expected at offset {self.i}")
            self._ws(False)
            if self.t.startswith("::=", self.i):
                self.i += 3
            elif self.t.startswith(":", self.i):
                self.i += 1
            else:
                raise GrammarError(f"'::=' expected after rule {name!r}")
            if name in rules:
                raise GrammarError(f"rule {name!r} defined twice")
            rules[name] = self._alternatives(top=True)
            self._ws()
        if not rules:
            raise GrammarError("empty grammar")
        return rules

    def _alternatives(self, top: bool) -> list:
        alts, cur = [], []
        while True:
            self._ws()
            if self.i >= len(self.t) or (top and self._at_rule_start()):
                break
            c = self.t[self.i]
            if c == "|":
                self.i += 1
                alts.append(cur)
                cur = []
                continue
            if c == ")":
                if top:
                    raise GrammarError(f"unbalanced ')' at offset {self.i}")
                break
            cur.append(self._postfix(self._item()))
        alts.append(cur)
        return alts

    def _item(self):
        c = self.t[self.i]
        if c in "\"'":
            j, out = self.i + 1, []
            while j < len(self.t) and self.t[j] != c:
                if self.t[j] == "\\" and j + 1 < len(self.t):
                    e = self.t[j + 1]
                    out.append({"n": "\n", "t": "\t", "r": "\r"}.get(e, e))
                    j += 2
                else:
                    out.append(self.t[j])
                    j += 1
            if j >= len(self.t):
                raise GrammarError("unterminated string literal")
            self.i = j + 1
            return ("lit", "".join(out))
        if c == "[":
            j = self.i + 1
            if j < len(self.t) and self.t[j] == "^":
                j += 1
            if j < len(self.t) and self.t[j] == "]":
                j += 1
            while j < len(self.t) and self.t[j] != "]":
                j += 2 if self.t[j] == "\\" else 1
            if j >= len(self.t):
                raise GrammarError("unterminated character class")
            src, self.i = self.t[self.i:j + 1], j + 1
            return ("class", src)
        if c == ".":
            self.i += 1
            return ("any",)
        if c == "(":
            self.i += 1
            alts = self._alternatives(top=False)
            if self.i >= len(self.t) or self.t[self.i] != ")":
                raise GrammarError("missing ')'")
            self.i += 1
            return ("group", alts)
        name = self._name()
        if name is None:
            raise GrammarError(f"unexpected {c!r} at offset {self.i}")
        return ("ref", name)

    def _postfix(self, item):
        while self.i < len(self.t):
            c = self.t[self.i]
            if c == "?":
                item, self.i = ("rep", item, 0, 1), self.i + 1
            elif c == "*":
                item, self.i = ("rep", item, 0, None), self.i + 1
            elif c == "+":
                item, self.i = ("rep", item, 1, None), self.i + 1
            elif c == "{":
                j = self.t.find("}", self.i)
                parts = self.t[self.i + 1:j].split(",") if j > 0 else []
                if not parts or not parts[0].strip().isdigit() or len(parts) > 2:
                    raise GrammarError(f"bad repetition at offset {self.i}")
                lo = int(parts[0])
                hi = lo if len(parts) == 1 else (int(parts[1]) if parts[1].strip() else None)
                item, self.i = ("rep", item, lo, hi), j + 1
            else:
                break
        return item


def grammar_to_regex(grammar: str, start: Optional[str] = None, max_depth: int = 3) -> str:
    """Regular expression of the strings a context-free grammar derives with every rule nested in itself at most
    ``max_depth`` times (the counterpart of the reference's ``guided_grammar``, which hands the grammar to xgrammar's
    pushdown automaton, vllm/v1/structured_output/backend_xgrammar.py; here the bounded language goes through the
    same DFA and token-mask machinery as regular expressions and JSON schemas). A derivation that would nest a rule
    deeper is left out; a grammar whose start rule has no derivation within the bound is an error. The start rule is
    ``start``, else ``root``, else the first rule."""
    rules = _GrammarParser(grammar).parse()
    if start is None:
        start = "root" if "root" in rules else ("start" if "start" in rules else next(iter(rules)))
    if start not in rules:
        raise GrammarError(f"no rule {start!r}")

    def alts_rx(alts, depth: dict) -> Optional[str]:
        out = []
        for items in alts:
            parts = []
            for it in items:
                r = item_rx(it, depth)
                if r is None:
                    parts = None
                    break
                parts.append(r)
            if parts is not None:
                out.append("".join(parts))
        if not out:
            return None
        return out[0] if len(out) == 1 else "(" + "|".join(out) + ")"

    def item_rx(it, depth: dict) -> Optional[str]:
        kind = it[0]
        if kind == "lit":
            return regex_escape(it[1])
        if kind == "class":
            return it[1]
        if kind == "any":
            return "."
        if kind == "group":
            r = alts_rx(it[1], depth)
            return None if r is None else "(" + r + ")"
        if kind == "ref":
            name = it[1]
            if name not in rules:
                raise GrammarError(f"rule {name!r} is used but not defined")
            d = depth.get(name, 0)
            if d > max_depth:
                return None
            depth[name] = d + 1
            r = alts_rx(rules[name], depth)
            depth[name] = d
            return None if r is None else "(" + r + ")"
        _, inner, lo, hi = it
        r = item_rx(inner, depth)
        if r is None:
            return "" if lo == 0 else None            # zero repetitions remain possible
        if (lo, hi) == (0, 1):
            return "(" + r + ")?"
        if (lo, hi) == (0, None):
            return "(" + r + ")*"
        if (lo, hi) == (1, None):
            return "(" + r + ")+"
        return "(" + r + "){" + str(lo) + ("" if hi == lo else "," + ("" if hi is None else str(hi))) + "}"

    rx = alts_rx(rules[start], {start: 1})
    if rx is None:
        raise GrammarError(f"rule {start!r} derives nothing within {max_depth} levels of nesting")
    if len(rx) > 200_000:
        raise GrammarError("the grammar unrolls into a regular expression that is too large; lower max_depth")
    return rx


def token_bytes_table(tokenizer, vocab_size: int) -> list[bytes]:
    """UTF-8 bytes every token contributes to the output text (empty for special / unknown tokens)."""
    if hasattr(tokenizer, "token_bytes"):
        return [tokenizer.token_bytes(i) for i in range(vocab_size)]
    special = set(getattr(tokenizer, "all_special_ids", []) or [])
    pieces = None
    if hasattr(tokenizer, "convert_ids_to_tokens"):
        try:
            pieces = tokenizer.convert_ids_to_tokens(list(range(vocab_size)))
        except Exception:
            pieces = None
    # byte-level BPE vocabularies (GPT-2 / Llama-3 / Qwen) spell every byte as one printable character
    printable = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    byte_of = {chr(b): b for b in printable}
    spare = 0
    for b in range(256):
        if b not in printable:
            byte_of[chr(256 + spare)] = b
            spare += 1
    byte_level = pieces is not None and any(p is not None and p.startswith("Ġ") for p in pieces[:50000])
    table = []
    for i in range(vocab_size):
        piece = pieces[i] if pieces is not None and i < len(pieces) else None
        if i in special or (pieces is not None and piece is None):
            table.append(b"")
        elif byte_level:
            table.append(bytes(byte_of[c] for c in piece) if all(c in byte_of for c in piece) else b"")
        elif len(piece) == 6 and piece.startswith("<0x") and piece.endswith(">"):
            table.append(bytes([int(piece[3:5], 16)]))             # sentencepiece byte fallback
        elif pieces is not None:
            table.append(piece.replace("▁", " ").encode("utf-8"))   # sentencepiece word-boundary marker
        else:
            try:
                text = tokenizer.decode([i], skip_special_tokens=False)
            except Exception:
                text = ""
            table.append(text.encode("utf-8") if "�" not in text else b"")
    return table


class TokenTrie:
    def __init__(self, table: Sequence[bytes]):
        self.vocab_size = len(table)
        self.root: dict = {}
        for tid, bs in enumerate(table):
            if not bs:
                continue
            node = self.root
            for b in bs:
                node = node.setdefault(b, {})
            node.setdefault(-1, []).append(tid)
        self.table = list(table)


class GuidedFSM:
    """A compiled constraint bound to a vocabulary: token masks per automaton state."""

    def __init__(self, dfa: DFA, trie: TokenTrie, eos_token_id: Optional[int], max_cached_states: int = 4096):
        self.dfa, self.trie, self.eos = dfa, trie, eos_token_id
        self._allowed: "OrderedDict[int, list[int]]" = OrderedDict()
        self._max = max_cached_states

    def state_after(self, token_ids: Sequence[int]) -> int:
        s = 0
        table = self.trie.table
        for t in token_ids:
            if t == self.eos:
                break
            s = self.dfa.walk(table[t] if 0 <= t < len(table) else b"", s)
            if s < 0:
                return -1
        return s

    def allowed_tokens(self, state: int) -> list[int]:
        """Token ids whose bytes keep the automaton alive from ``state`` (+ EOS in accepting states)."""
        got = self._allowed.get(state)
        if got is not None:
            self._allowed.move_to_end(state)
            return got
        out: list[int] = []
        if state >= 0:
            step = self.dfa.step
            stack = [(self.trie.root, state)]
            while stack:
                node, s = stack.pop()
                for b, child in node.items():
                    if b == -1:
                        continue
                    ns = step(s, b)
                    if ns < 0:
                        continue
                    ids = child.get(-1)
                    if ids:
                        out.extend(ids)
                    stack.append((child, ns))
            if self.dfa.accepting[state] and self.eos is not None:
                out.append(self.eos)
        out.sort()
        self._allowed[state] = out
        if len(self._allowed) > self._max:
            self._allowed.popitem(last=False)
        return out


_COMPILED: "OrderedDict[tuple, GuidedFSM]" = OrderedDict()


def constraint_pattern(sp) -> Optional[str]:
    """The regular expression a request's sampling parameters ask for (None: unconstrained)."""
    if getattr(sp, "guided_pattern", None):
        return sp.guided_pattern
    if getattr(sp, "guided_regex", None):
        return sp.guided_regex
    gj = getattr(sp, "guided_json", None)
    if gj is not None and gj is not False:
        return json_schema_to_regex(gj)
    gg = getattr(sp, "guided_grammar", None)
    if gg:
        return grammar_to_regex(gg)
    return None


def get_fsm(pattern: str, trie: TokenTrie, eos_token_id: Optional[int]) -> GuidedFSM:
    key = (pattern, id(trie), eos_token_id)
    fsm = _COMPILED.get(key)
    if fsm is None:
        fsm = GuidedFSM(DFA(pattern), trie, eos_token_id)
        _COMPILED[key] = fsm
        if len(_COMPILED) > 64:
            _COMPILED.popitem(last=False)
    else:
        _COMPILED.move_to_end(key)
    return fsm
