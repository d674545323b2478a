"""Tokenisation and incremental detokenisation (vllm/v1/engine/processor.py, detokenizer.py).

A HuggingFace tokenizer directory is used when given; ``ByteTokenizer`` (UTF-8 bytes + BOS/EOS) is a
dependency-free stand-in for offline tests and random-weight runs."""
from __future__ import annotations

from typing import Optional


class ByteTokenizer:
    """ids 0..255 = bytes, 256 = BOS, 257 = EOS; any larger id decodes to U+FFFD."""
    bos_token_id = 256
    eos_token_id = 257
    vocab_size = 258

    def token_bytes(self, token_id: int) -> bytes:
        """The bytes a token adds to the output text (structured output walks these)."""
        return bytes([token_id]) if 0 <= token_id < 256 else b""

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        out = bytearray()
        pieces = []
        for t in ids:
            if t < 256:
                out.append(t)
            else:
                if out:
                    pieces.append(out.decode("utf-8", errors="replace"))
                    out = bytearray()
                if t > 257 or not skip_special_tokens:
                    pieces.append("�" if t > 257 else ("<s>" if t == 256 else "</s>"))
        if out:
            pieces.append(out.decode("utf-8", errors="replace"))
        return "".join(pieces)


def load_tokenizer(name_or_path: Optional[str]):
    if name_or_path in (None, "byte"):
        return ByteTokenizer()
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(name_or_path)


class IncrementalDetokenizer:
    """Keeps the text of a request up to date as tokens arrive and checks stop strings."""

    def __init__(self, tokenizer, prompt_ids: list[int], skip_special_tokens: bool = True,
                 stop: Optional[list[str]] = None, include_stop: bool = False):
        self.tokenizer = tokenizer
        self.skip_special = skip_special_tokens
        self.stop = stop or []
        self.include_stop = include_stop     # keep the matched stop string at the end of the text
        self.token_ids: list[int] = []
        self.text = ""
        self._emitted_prefix = 0     # tokens already turned into stable text
        self._read = 0

    def update(self, new_ids: list[int]) -> Optional[str]:
        """Append tokens; returns the stop string that now terminates the text, if any."""
        self.token_ids.extend(new_ids)
        # decode from a small window back so multi-token characters come out right
        start = max(0, self._emitted_prefix - 6)
        window_old = self.tokenizer.decode(self.token_ids[start:self._emitted_prefix], skip_special_tokens=self.skip_special)
        window_new = self.tokenizer.decode(self.token_ids[start:], skip_special_tokens=self.skip_special)
        if window_new.endswith("�"):
            return None              # incomplete UTF-8 sequence: wait for the next token
        delta = window_new[len(window_old):]
        self.text += delta
        self._emitted_prefix = len(self.token_ids)
        for s in self.stop:
            # a new match must touch the text that was just added
            pos = self.text.find(s, max(0, len(self.text) - len(delta) - len(s) + 1))
            if pos >= 0:
                self.text = self.text[:pos + (len(s) if self.include_stop else 0)]
                return s
        return None
