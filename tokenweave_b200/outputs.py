"""Result types returned by ``LLM.generate`` (counterpart of vllm/outputs.py)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class CompletionOutput:
    index: int
    text: str
    token_ids: list[int]
    cumulative_logprob: Optional[float] = None
    logprobs: Optional[list[dict[int, float]]] = None
    finish_reason: Optional[str] = None   # "stop" | "length" | "abort"
    stop_reason: Optional[object] = None

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclass
class RequestMetrics:
    arrival_time: float = 0.0
    first_scheduled_time: Optional[float] = None
    first_token_time: Optional[float] = None
    finished_time: Optional[float] = None


@dataclass
class RequestOutput:
    request_id: str
    prompt: Optional[str]
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput]
    finished: bool
    metrics: RequestMetrics = field(default_factory=RequestMetrics)
    # with ``SamplingParams.prompt_logprobs``: one entry per prompt token, None for the first, then
    # ``{token id: log-probability}`` holding the prompt token itself and the k most likely tokens there
    prompt_logprobs: Optional[list] = None
    pooled: Optional[object] = None      # with ``SamplingParams.pooling``: fp32 hidden state (host tensor)


@dataclass
class BeamSearchSequence:
    """One hypothesis of ``LLM.beam_search``: prompt + generated token ids and their summed log-probability."""
    tokens: list[int]
    cum_logprob: float = 0.0
    text: Optional[str] = None


@dataclass
class BeamSearchOutput:
    sequences: list[BeamSearchSequence]


@dataclass
class PoolingOutput:
    """Result of ``LLM.encode`` / ``LLM.embed``: ``data`` is the pooled hidden state (fp32, on the host)."""
    request_id: str
    prompt_token_ids: list[int]
    data: "object"


@dataclass
class ClassificationOutput:
    """Result of ``LLM.classify``: class probabilities from the checkpoint's sequence-classification head."""
    request_id: str
    prompt_token_ids: list[int]
    probs: list[float]
