"""Sampling parameters of a request (subset of vllm/sampling_params.py used by offline inference)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Union


@dataclass
class SamplingParams:
    n: int = 1
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    stop: Union[None, str, list[str]] = None
    stop_token_ids: Optional[list[int]] = None
    include_stop_str_in_output: bool = False
    max_tokens: Optional[int] = 16
    min_tokens: int = 0
    ignore_eos: bool = False
    logprobs: Optional[int] = None
    # log-probability of every prompt token given its prefix, plus the k most likely tokens at each position
    # (vllm/sampling_params.py ``prompt_logprobs``); such a request does not reuse cached prefixes
    prompt_logprobs: Optional[int] = None
    # pooling request: the final-norm hidden state at the last prompt token comes back in
    # ``RequestOutput.pooled`` (what ``LLM.encode`` and the server's embedding endpoint use)
    pooling: bool = False
    truncate_prompt_tokens: Optional[int] = None      # keep only the last k prompt tokens
    detokenize: bool = True
    skip_special_tokens: bool = True
    logit_bias: Optional[dict] = None                   # token id -> additive bias (clamped to [-100, 100])
    allowed_token_ids: Optional[list[int]] = None       # every other token is masked out
    bad_words_token_ids: Optional[list[list[int]]] = None   # token sequences that must not be generated
    eos_token_id: Optional[int] = None                  # filled in by the engine; masked while below min_tokens
    # Constrained decoding to one of several strings (the "choice" mode of the reference's guided decoding,
    # vllm/sampling_params.py ``GuidedDecodingParams.choice``): texts here, tokenised by the engine into
    # ``guided_choice_token_ids``; generation stops when a choice is complete.
    guided_choice: Optional[list[str]] = None
    guided_choice_token_ids: Optional[list[list[int]]] = None
    # Structured output (``GuidedDecodingParams.regex`` / ``.json`` of the reference): the generated text must
    # match the regular expression, or be a JSON document satisfying the schema (a dict or its JSON text;
    # ``{}`` admits any JSON value). The engine lowers both to ``guided_pattern``; see engine/structured.py.
    guided_regex: Optional[str] = None
    guided_json: Union[None, str, dict] = None
    # a context-free grammar (GBNF / EBNF text); served with every rule nested in itself a bounded number of times
    guided_grammar: Optional[str] = None
    guided_pattern: Optional[str] = None

    def __post_init__(self):
        if self.logit_bias is not None:
            self.logit_bias = {int(k): max(-100.0, min(100.0, float(v))) for k, v in self.logit_bias.items()}
        if self.allowed_token_ids is not None and not self.allowed_token_ids:
            raise ValueError("allowed_token_ids must not be empty")
        if self.bad_words_token_ids is not None and any(len(w) == 0 for w in self.bad_words_token_ids):
            raise ValueError("bad_words_token_ids must not contain empty sequences")
        if isinstance(self.stop, str):
            self.stop = [self.stop]
        self.stop = list(self.stop or [])
        self.stop_token_ids = list(self.stop_token_ids or [])
        if self.truncate_prompt_tokens is not None and self.truncate_prompt_tokens < 1:
            raise ValueError("truncate_prompt_tokens must be at least 1")
        if self.n < 1:
            raise ValueError("n must be at least 1")
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < -1 or self.top_k == 0:
            raise ValueError("top_k must be -1 (disabled) or positive")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-5

    @property
    def needs_penalties(self) -> bool:
        """True when the logits must be edited before sampling (penalties, biases, masks)."""
        return (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or self.repetition_penalty != 1.0
                or bool(self.logit_bias) or self.allowed_token_ids is not None or bool(self.bad_words_token_ids)
                or self.min_tokens > 0 or bool(self.guided_choice_token_ids)
                or bool(self.guided_regex) or self.guided_json is not None or bool(self.guided_grammar)
                or bool(self.guided_pattern))

    def clone(self) -> "SamplingParams":
        import copy
        return copy.deepcopy(self)


@dataclass
class BeamSearchParams:
    """Parameters of ``LLM.beam_search`` (vllm/sampling_params.py ``BeamSearchParams``)."""
    beam_width: int
    max_tokens: int
    ignore_eos: bool = False
    temperature: float = 0.0
    length_penalty: float = 1.0

    def __post_init__(self):
        if self.beam_width < 1 or self.max_tokens < 1:
            raise ValueError("beam_width and max_tokens must be at least 1")
