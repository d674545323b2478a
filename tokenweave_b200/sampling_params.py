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
    max_tokens: Optional[int] = 16
    min_tokens: int = 0
    ignore_eos: bool = False
    logprobs: Optional[int] = None
    detokenize: bool = True
    skip_special_tokens: bool = True

    def __post_init__(self):
        if isinstance(self.stop, str):
            self.stop = [self.stop]
        self.stop = list(self.stop or [])
        self.stop_token_ids = list(self.stop_token_ids or [])
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
        return (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or self.repetition_penalty != 1.0)

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
