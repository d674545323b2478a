"""Per-request engine state (counterpart of vllm/v1/request.py)."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Optional

from ..sampling_params import SamplingParams


class RequestStatus(enum.IntEnum):
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2
    FINISHED_STOPPED = 3
    FINISHED_LENGTH = 4
    FINISHED_ABORTED = 5

    @property
    def finished(self) -> bool:
        return self >= RequestStatus.FINISHED_STOPPED


FINISH_REASON = {RequestStatus.FINISHED_STOPPED: "stop", RequestStatus.FINISHED_LENGTH: "length",
                 RequestStatus.FINISHED_ABORTED: "abort"}


@dataclass(eq=False)        # identity semantics: membership tests in the queues must not compare token lists
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    eos_token_id: Optional[int] = None
    arrival_time: float = field(default_factory=time.monotonic)
    prompt: Optional[str] = None

    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list[int] = field(default_factory=list)
    num_computed_tokens: int = 0       # tokens whose KV is in the cache
    block_ids: list[int] = field(default_factory=list)
    spec_token_ids: list[int] = field(default_factory=list)   # drafts to verify in the next step
    lora_request: Optional[object] = None                     # tokenweave_b200.lora.LoRARequest
    prompt_logprobs: dict = field(default_factory=dict)       # prompt position -> {token id: log-probability}
    priority: int = 0                                         # scheduling_policy="priority": lower values first
    pooled: Optional[object] = None                           # pooling requests: hidden state at the last prompt token
    block_hash_chain: list = field(default_factory=list)      # prefix-cache hashes of the full blocks so far
    num_published_blocks: int = 0                             # leading blocks already offered to the prefix cache
    stop_reason: Optional[object] = None
    first_scheduled_time: Optional[float] = None
    first_token_time: Optional[float] = None
    finished_time: Optional[float] = None

    @property
    def cache_salt(self) -> bytes:
        """Prefix-cache key component: KV computed under one adapter is not valid under another."""
        return b"" if self.lora_request is None else f"lora{self.lora_request.lora_int_id}|".encode()

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    def token_at(self, i: int) -> int:
        n = len(self.prompt_token_ids)
        return self.prompt_token_ids[i] if i < n else self.output_token_ids[i - n]

    @property
    def finish_reason(self) -> Optional[str]:
        return FINISH_REASON.get(self.status)
