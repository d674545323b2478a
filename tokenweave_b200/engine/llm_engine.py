"""Engine front end: tokenises requests, drives the core, turns tokens back into ``RequestOutput``s.

Counterpart of vllm/v1/engine/llm_engine.py:41-231, processor.py and output_processor.py (n > 1 fan-out,
incremental detokenisation, stop strings).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional, Union

from ..config import EngineArgs, EngineConfig
from ..outputs import CompletionOutput, RequestMetrics, RequestOutput
from ..sampling_params import SamplingParams
from ..utils.logging import init_logger
from ..utils.metrics import LoggingStatLogger
from .core import EngineCore
from .request import Request, RequestStatus
from .tokenizer import IncrementalDetokenizer, load_tokenizer

logger = init_logger(__name__)


@dataclass
class _Parent:
    request_id: str
    prompt: Optional[str]
    prompt_token_ids: list[int]
    params: SamplingParams
    children: list[Request] = field(default_factory=list)
    detoks: list[Optional[IncrementalDetokenizer]] = field(default_factory=list)
    logprobs: list[list] = field(default_factory=list)
    cum_logprob: list[float] = field(default_factory=list)
    arrival: float = field(default_factory=time.monotonic)


class LLMEngine:
    def __init__(self, config: EngineConfig, executor=None):
        self.config = config
        self.tokenizer = None if config.skip_tokenizer_init else load_tokenizer(config.tokenizer or
                                                                               (config.model.path if config.model.path else "byte"))
        if config.engine_core_process and executor is None:
            from .core_client import MPEngineCoreClient
            self.core = MPEngineCoreClient(config)
        else:
            self.core = EngineCore(config, executor)
        self.parents: dict[str, _Parent] = {}
        self.child_to_parent: dict[str, tuple[str, int]] = {}
        self.stat_logger = None if config.disable_log_stats else LoggingStatLogger()
        eos = config.model.eos_token_id
        if eos is None and self.tokenizer is not None:
            eos = getattr(self.tokenizer, "eos_token_id", None)
        self.eos_token_id = eos

    @classmethod
    def from_engine_args(cls, args: EngineArgs) -> "LLMEngine":
        return cls(args.create_engine_config())

    # ---- requests ---------------------------------------------------------------------------
    def add_request(self, request_id: str, prompt: Union[str, list[int], dict], params: SamplingParams,
                    lora_request=None, priority: int = 0) -> None:
        if lora_request is not None and not self.config.enable_lora:
            raise ValueError("pass enable_lora=True to serve LoRA adapters")
        text: Optional[str] = None
        if isinstance(prompt, dict):
            text = prompt.get("prompt")
            ids = prompt.get("prompt_token_ids")
            if ids is None:
                ids = self._encode(text)
        elif isinstance(prompt, str):
            text, ids = prompt, self._encode(prompt)
        else:
            ids = list(prompt)
        if params.truncate_prompt_tokens is not None:
            ids = list(ids)[-params.truncate_prompt_tokens:]        # keep the end of the prompt (left truncation)
        vocab = self.config.model.vocab_size
        if any((t < 0 or t >= vocab) for t in ids):
            raise ValueError(f"request {request_id}: token id outside [0, {vocab})")
        parent = _Parent(request_id, text, list(ids), params)
        for i in range(params.n):
            sp = params
            if params.n > 1:
                sp = params.clone()
                sp.n = 1
                if sp.seed is not None:
                    sp.seed = sp.seed + i
            if sp.guided_choice and not sp.guided_choice_token_ids:
                if self.tokenizer is None:
                    raise ValueError("guided_choice needs a tokenizer (or pass guided_choice_token_ids)")
                if sp is params:
                    sp = params.clone()
                sp.guided_choice_token_ids = [list(self.tokenizer.encode(c, add_special_tokens=False))
                                              for c in sp.guided_choice]
                sp.eos_token_id = self.eos_token_id
            if (sp.guided_regex or sp.guided_json is not None or sp.guided_grammar) and not sp.guided_pattern:
                from . import structured
                if self.eos_token_id is None:
                    raise ValueError("structured output ends a request through the end-of-sequence token; "
                                     "the model configuration or tokenizer must define one")
                if sp is params:
                    sp = params.clone()
                sp.guided_pattern = structured.constraint_pattern(sp)
                structured.DFA(sp.guided_pattern)          # syntax errors surface here, not on the workers
                sp.eos_token_id = self.eos_token_id
                sp.ignore_eos = False
            if sp.min_tokens > 0 and sp.eos_token_id is None and not sp.ignore_eos:
                if sp is params:
                    sp = params.clone()          # the caller's object stays untouched
                sp.eos_token_id = self.eos_token_id     # the sampler masks it until min_tokens is reached
            cid = request_id if params.n == 1 else f"{i}_{request_id}"
            child = Request(cid, list(ids), sp, eos_token_id=self.eos_token_id, prompt=text, lora_request=lora_request,
                            priority=priority)
            parent.children.append(child)
            detok = None
            if self.tokenizer is not None and params.detokenize:
                detok = IncrementalDetokenizer(self.tokenizer, ids, params.skip_special_tokens, params.stop,
                                               params.include_stop_str_in_output)
            parent.detoks.append(detok)
            parent.logprobs.append([])
            parent.cum_logprob.append(0.0)
            self.child_to_parent[cid] = (request_id, i)
            self.core.add_request(child)
        self.parents[request_id] = parent

    def tokenize_prompt(self, prompt: Union[str, list[int], dict]) -> list[int]:
        """Token ids of a prompt given as text, ids, or a ``{"prompt" / "prompt_token_ids"}`` dict."""
        if isinstance(prompt, dict):
            ids = prompt.get("prompt_token_ids")
            return list(ids) if ids is not None else self._encode(prompt.get("prompt"))
        return self._encode(prompt) if isinstance(prompt, str) else list(prompt)

    def _encode(self, text: str) -> list[int]:
        if self.tokenizer is None:
            raise ValueError("text prompts need a tokenizer (skip_tokenizer_init is set)")
        return list(self.tokenizer.encode(text))

    def abort_request(self, request_id: str) -> None:
        parent = self.parents.pop(request_id, None)
        if parent:
            for c in parent.children:
                self.core.abort_request(c.request_id)
                self.child_to_parent.pop(c.request_id, None)

    def has_unfinished_requests(self) -> bool:
        return self.core.has_unfinished_requests()

    def get_num_unfinished_requests(self) -> int:
        return self.core.scheduler.num_unfinished()

    # ---- stepping ---------------------------------------------------------------------------
    def step(self, final_only: bool = False) -> list[RequestOutput]:
        """One engine iteration. Returns a snapshot of every request that produced a token or finished;
        with ``final_only`` only finished requests are materialised (what the offline API consumes —
        the counterpart of ``RequestOutputKind.FINAL_ONLY`` in vllm/sampling_params.py), which keeps the
        per-step host cost independent of the lengths generated so far."""
        touched = self.core.step()
        if self.stat_logger is not None and self.core.last_stats is not None:
            self.stat_logger.record(self.core.last_stats)
        lps = getattr(self.core, "_last_logprobs", {})
        outputs: dict[str, RequestOutput] = {}
        for child in touched:
            pid, idx = self.child_to_parent[child.request_id]
            parent = self.parents[pid]
            lp = lps.get(child.request_id)
            if lp is not None:
                parent.logprobs[idx].append(lp)
                parent.cum_logprob[idx] += lp.get(child.output_token_ids[-1], 0.0)
            detok = parent.detoks[idx]
            if detok is not None and not child.status == RequestStatus.FINISHED_ABORTED:
                hit = detok.update(child.output_token_ids[len(detok.token_ids):])
                if hit is not None and not child.status.finished:
                    self.core.scheduler.finish_request(child, RequestStatus.FINISHED_STOPPED, hit)
            outputs[pid] = parent
        if final_only:
            outputs = {pid: p for pid, p in outputs.items() if all(c.status.finished for c in p.children)}
        outputs = {pid: self._make_output(p) for pid, p in outputs.items()}
        done = [pid for pid, out in outputs.items() if out.finished]
        for pid in done:
            parent = self.parents.pop(pid)
            for c in parent.children:
                self.child_to_parent.pop(c.request_id, None)
        return list(outputs.values())

    def _make_output(self, parent: _Parent) -> RequestOutput:
        comps = []
        for i, c in enumerate(parent.children):
            detok = parent.detoks[i]
            comps.append(CompletionOutput(
                index=i, text=detok.text if detok is not None else "", token_ids=list(c.output_token_ids),
                cumulative_logprob=parent.cum_logprob[i] if parent.params.logprobs is not None else None,
                logprobs=list(parent.logprobs[i]) if parent.params.logprobs is not None else None,
                finish_reason=c.finish_reason, stop_reason=c.stop_reason))
        finished = all(c.status.finished for c in parent.children)
        first = [c.first_token_time for c in parent.children if c.first_token_time is not None]
        metrics = RequestMetrics(parent.arrival, min((c.first_scheduled_time or parent.arrival) for c in parent.children),
                                 min(first) if first else None,
                                 max((c.finished_time or 0.0) for c in parent.children) if finished else None)
        plp = None
        if parent.params.prompt_logprobs is not None:
            got = parent.children[0].prompt_logprobs        # the children share the prompt
            plp = [None] + [got.get(p) for p in range(1, len(parent.prompt_token_ids))]
        return RequestOutput(parent.request_id, parent.prompt, parent.prompt_token_ids, comps, finished, metrics,
                             prompt_logprobs=plp, pooled=parent.children[0].pooled)

    def shutdown(self) -> None:
        self.core.shutdown()
