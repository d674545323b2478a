"""Speculative decoding with an n-gram (prompt-lookup) proposer.

Counterpart of vllm/v1/spec_decode/ngram_proposer.py and the verification path of
vllm/v1/worker/gpu_model_runner.py / vllm/v1/sample/rejection_sampler.py, for greedy requests: after
every step the engine looks the request's last ``n`` tokens up in its own history (prompt + output) and
proposes the ``k`` tokens that followed the most recent earlier occurrence; the next step runs the last
sampled token and the ``k`` drafts through the model as one ``k + 1``-token query, takes the argmax at
every position, keeps the drafts that equal the model's choice and one more token (the model's choice
after the last accepted draft). The output is token-for-token what plain greedy decoding produces; a
step yields between 1 and ``k + 1`` tokens. The KV entries of rejected drafts are simply overwritten
by the next step (slots are addressed by position).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence


@dataclass
class SpecDecodeConfig:
    num_speculative_tokens: int = 0        # k; 0 disables
    prompt_lookup_max: int = 4             # longest suffix n-gram tried
    prompt_lookup_min: int = 2             # shortest

    @property
    def enabled(self) -> bool:
        return self.num_speculative_tokens > 0

    @staticmethod
    def from_user(value) -> "SpecDecodeConfig":
        """``None``, an int (k), or the reference's ``speculative_config`` dict
        ``{"method": "ngram", "num_speculative_tokens": k, "prompt_lookup_max": n, "prompt_lookup_min": m}``."""
        if value is None:
            return SpecDecodeConfig()
        if isinstance(value, SpecDecodeConfig):
            return value
        if isinstance(value, int):
            return SpecDecodeConfig(num_speculative_tokens=value)
        if isinstance(value, dict):
            method = value.get("method", "ngram")
            if method not in ("ngram", "[ngram]"):
                raise ValueError(f"speculative method {method!r} is not supported (only 'ngram')")
            hi = int(value.get("prompt_lookup_max", 4))
            lo = int(value.get("prompt_lookup_min", min(2, hi)))
            if not 1 <= lo <= hi:
                raise ValueError("need 1 <= prompt_lookup_min <= prompt_lookup_max")
            return SpecDecodeConfig(int(value.get("num_speculative_tokens", 0)), hi, lo)
        raise TypeError("speculative_config must be None, an int or a dict")


def ngram_propose(token_ids: Sequence[int], k: int, max_n: int = 4, min_n: int = 2) -> list[int]:
    """Up to ``k`` draft tokens: the continuation of the most recent earlier occurrence of the longest
    suffix n-gram (``max_n`` down to ``min_n``) of ``token_ids``; empty when nothing matches."""
    L = len(token_ids)
    if k <= 0 or L < min_n + 1:
        return []
    for n in range(min(max_n, L - 1), min_n - 1, -1):
        suffix = list(token_ids[L - n:])
        # most recent earlier start i with token_ids[i:i+n] == suffix and at least one token after it
        for i in range(L - n - 1, -1, -1):
            if token_ids[i] == suffix[0] and list(token_ids[i:i + n]) == suffix:
                cont = list(token_ids[i + n:i + n + k])
                if cont:
                    return cont
    return []


def accept_greedy(drafts: Sequence[int], targets: Sequence[int]) -> list[int]:
    """``targets[i]`` is the model's greedy choice after the last sampled token and ``drafts[:i]``
    (``len(targets) == len(drafts) + 1``). Returns the tokens this step emits: the accepted drafts and
    the model's choice at the first disagreement (or after the last draft)."""
    out: list[int] = []
    for i, d in enumerate(drafts):
        if int(targets[i]) != int(d):
            out.append(int(targets[i]))
            return out
        out.append(int(d))
    out.append(int(targets[len(drafts)]))
    return out


def spec_eligible(sampling_params) -> bool:
    """Greedy requests without penalties or log-probabilities can be verified by plain argmax."""
    sp = sampling_params
    return sp.greedy and not sp.needs_penalties and sp.logprobs is None


def clamp_drafts(drafts: list[int], num_tokens: int, max_model_len: int, max_tokens: Optional[int],
                 num_output_tokens: int) -> list[int]:
    """Never draft past the context window or the request's own token limit."""
    room = max_model_len - 1 - num_tokens
    if max_tokens is not None:
        room = min(room, max_tokens - num_output_tokens - 1)
    return drafts[:max(0, room)]
