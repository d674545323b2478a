"""Continuous-batching scheduler with a per-step token budget (chunked prefill by construction).

Counterpart of vllm/v1/core/sched/scheduler.py:133-498 (schedule) and :609-735 (update_from_output):
running requests are served first, then waiting ones, each capped by what is left of
``max_num_batched_tokens``; a request whose prompt does not fit is prefetched in chunks; when the
KV pool is exhausted the most recently admitted running request is preempted and recomputed later.
The schedule is a pure function of the request stream, so SPMD ranks that replay the same calls
stay in lockstep without exchanging messages.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..config import SchedulerConfig
from .kv_cache import KVCacheManager
from .request import Request, RequestStatus


@dataclass
class ScheduledRequest:
    request: Request
    num_new_tokens: int
    num_computed_tokens: int     # before this step
    is_new: bool                 # first time (or resumed after preemption) on the workers
    spec_token_ids: list[int] = field(default_factory=list)   # drafts verified in this step (the last tokens)


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledRequest] = field(default_factory=list)
    total_num_tokens: int = 0
    finished_req_ids: list[str] = field(default_factory=list)
    preempted_req_ids: list[str] = field(default_factory=list)
    step_id: int = 0
    # KV connector: (block id, block hash) pairs the workers fill from the external store before the step runs
    kv_loads: list = field(default_factory=list)

    @property
    def empty(self) -> bool:
        return self.total_num_tokens == 0


@dataclass
class ModelRunnerOutput:
    req_ids: list[str]
    # None for requests still prefilling; an int, or (speculative decoding) the list of tokens the step emitted
    sampled_token_ids: list
    logprobs: Optional[list] = None


class Scheduler:
    def __init__(self, config: SchedulerConfig, kv: KVCacheManager, spec=None):
        from .spec_decode import SpecDecodeConfig
        self.config = config
        self.kv = kv
        self.spec = spec if spec is not None else SpecDecodeConfig()
        self.connector = None              # engine.kv_connector.SharedStorageConnector of a consuming engine
        self.num_draft_tokens = 0          # statistics of speculative decoding
        self.num_accepted_tokens = 0
        self.last_emitted = 0
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.requests: dict[str, Request] = {}
        self._finished_since_last: list[str] = []
        self._step = 0

    # ---- request lifecycle -------------------------------------------------------------
    def add_request(self, req: Request) -> None:
        if req.num_prompt_tokens == 0:
            raise ValueError("empty prompt")
        if req.num_prompt_tokens >= self.config.max_model_len:
            raise ValueError(f"prompt of {req.num_prompt_tokens} tokens does not fit max_model_len "
                             f"{self.config.max_model_len}")
        if self.config.policy not in ("fcfs", "priority"):
            raise ValueError(f"unknown scheduling policy {self.config.policy!r}")
        self.requests[req.request_id] = req
        if self.config.policy == "priority":
            # keep the queue ordered by (priority, arrival); vllm/v1/core/sched/scheduler.py "priority" policy
            i = len(self.waiting)
            while i > 0 and self.waiting[i - 1].priority > req.priority:
                i -= 1
            self.waiting.insert(i, req)
        else:
            self.waiting.append(req)

    def abort_request(self, request_id: str) -> None:
        req = self.requests.get(request_id)
        if req is None or req.status.finished:
            return
        if req in self.running:
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        self._finish(req, RequestStatus.FINISHED_ABORTED)

    def has_unfinished_requests(self) -> bool:
        return bool(self.waiting or self.running)

    def num_unfinished(self) -> int:
        return len(self.waiting) + len(self.running)

    # ---- scheduling ---------------------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput(step_id=self._step)
        self._step += 1
        budget = self.config.max_num_batched_tokens
        cap = self.config.long_prefill_token_threshold
        preempted: list[Request] = []

        # running requests first (decode tokens and prefill continuations)
        i = 0
        while i < len(self.running) and budget > 0:
            req = self.running[i]
            n = min(req.num_tokens - req.num_computed_tokens, budget)
            if 0 < cap < n and self.config.enable_chunked_prefill:
                n = cap
            if not self.config.enable_chunked_prefill and n < req.num_tokens - req.num_computed_tokens:
                i += 1
                continue
            drafts: list[int] = []
            if req.spec_token_ids:
                # a decoding request (one uncomputed token) takes its drafts along as extra query tokens
                if n == 1 and req.num_tokens - req.num_computed_tokens == 1:
                    drafts = req.spec_token_ids[:max(0, budget - n)]
                    n += len(drafts)
                req.spec_token_ids = []
            while not self.kv.allocate_slots(req, n):
                if self.config.policy == "priority":
                    # the least urgent running request goes first, the most recently admitted among equals
                    worst = max(range(len(self.running)), key=lambda j: (self.running[j].priority, j))
                    victim = self.running.pop(worst)
                    if worst < i:
                        i -= 1                  # the list shifted under the cursor
                        # the victim already has its tokens in this step: take them out again (its blocks are
                        # about to be freed) and hand the tokens back to the budget
                        for k, sr in enumerate(out.scheduled):
                            if sr.request is victim:
                                budget += sr.num_new_tokens
                                del out.scheduled[k]
                                break
                else:
                    victim = self.running.pop()     # most recently admitted
                self._preempt(victim)
                preempted.append(victim)
                if victim is req:
                    n = 0
                    break
            if n == 0:
                break
            out.scheduled.append(ScheduledRequest(req, n, req.num_computed_tokens, False, drafts))
            budget -= n
            i += 1

        # then admit waiting requests
        if not preempted:
            while self.waiting and budget > 0 and len(self.running) < self.config.max_num_seqs:
                req = self.waiting[0]
                cached, n_cached = ([], 0)
                if req.num_computed_tokens == 0 and req.sampling_params.prompt_logprobs is None:
                    # (prompt log-probabilities need the hidden state of every prompt position: no cache hits)
                    cached, n_cached = self.kv.get_computed_blocks(req)
                # blocks the local cache does not have may be in the external store (the hook of
                # vllm/v1/core/sched/scheduler.py:319-367): they are loaded into fresh blocks before the step
                ext_hashes: list = []
                if (self.connector is not None and req.num_computed_tokens == 0
                        and req.sampling_params.prompt_logprobs is None):
                    want = self.kv.prefix_hashes(req)[len(cached):]
                    ext_hashes = want[:self.connector.num_matched(want)]
                n_ext = len(ext_hashes) * self.kv.block_size
                remaining = req.num_tokens - req.num_computed_tokens - n_cached - n_ext
                n = min(remaining, budget)
                if 0 < cap < n and self.config.enable_chunked_prefill:
                    n = cap
                if n < remaining and not self.config.enable_chunked_prefill:
                    break
                req.num_computed_tokens += n_cached
                if not self.kv.allocate_slots(req, n_ext + n, cached):
                    req.num_computed_tokens -= n_cached
                    break
                for j, h in enumerate(ext_hashes):
                    out.kv_loads.append((req.block_ids[len(cached) + j], h))
                req.num_computed_tokens += n_ext
                self.waiting.popleft()
                req.status = RequestStatus.RUNNING
                if req.first_scheduled_time is None:
                    req.first_scheduled_time = time.monotonic()
                self.running.append(req)
                out.scheduled.append(ScheduledRequest(req, n, req.num_computed_tokens, True))
                budget -= n

        out.total_num_tokens = sum(s.num_new_tokens for s in out.scheduled)
        out.finished_req_ids = self._finished_since_last
        self._finished_since_last = []
        out.preempted_req_ids = [r.request_id for r in preempted]
        return out

    def _preempt(self, req: Request) -> None:
        self.kv.free(req)
        req.status = RequestStatus.PREEMPTED
        req.num_computed_tokens = 0
        req.spec_token_ids = []
        self.waiting.appendleft(req)

    # ---- results ------------------------------------------------------------------------
    def update_from_output(self, sched: SchedulerOutput, result: ModelRunnerOutput) -> list[Request]:
        """Advance every scheduled request; returns the requests that produced a token or finished."""
        sampled = dict(zip(result.req_ids, result.sampled_token_ids))
        touched: list[Request] = []
        self.last_emitted = 0              # tokens appended to outputs by this step
        spec_on = self.spec.enabled
        for s in sched.scheduled:
            req = s.request
            if req.status.finished:
                continue
            tok = sampled.get(req.request_id)
            if not s.spec_token_ids and type(tok) is int and not spec_on:
                # the common decode step (one sampled token, no drafts): the general path below without its
                # temporaries and helper calls
                req.num_computed_tokens = s.num_computed_tokens + s.num_new_tokens
                if req.num_computed_tokens < req.num_tokens:
                    self.kv.cache_full_blocks(req)
                    continue
                req.output_token_ids.append(tok)
                self.last_emitted += 1
                if req.first_token_time is None:
                    req.first_token_time = time.monotonic()
                stop = self._stop_decision(req)
                self.kv.cache_full_blocks(req)
                if stop is not None:
                    self._stop_running(req, *stop)
                touched.append(req)
                continue
            toks = [int(t) for t in tok] if isinstance(tok, (list, tuple)) else ([] if tok is None else [int(tok)])
            # drafts that the model did not confirm leave no valid KV behind: they are not "computed"
            rejected = 0
            if s.spec_token_ids:
                accepted = max(0, len(toks) - 1)
                rejected = len(s.spec_token_ids) - accepted
                self.num_draft_tokens += len(s.spec_token_ids)
                self.num_accepted_tokens += accepted
            req.num_computed_tokens = s.num_computed_tokens + s.num_new_tokens - rejected
            if req.num_computed_tokens - (len(toks) - 1 if s.spec_token_ids else 0) < req.num_tokens or not toks:
                self.kv.cache_full_blocks(req)
                continue                       # still prefilling: the sampled token (if any) is discarded
            stop = None
            for t in toks:
                req.output_token_ids.append(t)
                self.last_emitted += 1
                if req.first_token_time is None:
                    req.first_token_time = time.monotonic()
                stop = self._stop_decision(req)
                if stop is not None:
                    break                      # tokens the step produced beyond a stop are dropped
            req.num_computed_tokens = min(req.num_computed_tokens, req.num_tokens)
            self.kv.cache_full_blocks(req)     # while the request still owns its blocks
            if stop is not None:
                self._stop_running(req, *stop)
            else:
                self._propose_drafts(req)
            touched.append(req)
        return touched

    def _propose_drafts(self, req: Request) -> None:
        """n-gram drafts for the next step of a greedy decoding request (empty when nothing matches)."""
        if not self.spec.enabled:
            return
        from .spec_decode import clamp_drafts, ngram_propose, spec_eligible
        if not spec_eligible(req.sampling_params):
            return
        drafts = ngram_propose(req.all_token_ids, self.spec.num_speculative_tokens, self.spec.prompt_lookup_max,
                               self.spec.prompt_lookup_min)
        req.spec_token_ids = clamp_drafts(drafts, req.num_tokens, self.config.max_model_len,
                                          req.sampling_params.max_tokens, len(req.output_token_ids))

    def _stop_decision(self, req: Request):
        """(status, stop_reason) if the request's last token ends it, else None. No side effects."""
        sp = req.sampling_params
        last = req.output_token_ids[-1]
        n_out = len(req.output_token_ids)
        if n_out >= sp.min_tokens:
            if not sp.ignore_eos and req.eos_token_id is not None and last == req.eos_token_id:
                return RequestStatus.FINISHED_STOPPED, None
            if last in sp.stop_token_ids:
                return RequestStatus.FINISHED_STOPPED, last
        if sp.guided_choice_token_ids:
            out = req.output_token_ids
            done = any(list(c) == out for c in sp.guided_choice_token_ids)
            longer = any(len(c) > len(out) and list(c[:len(out)]) == out for c in sp.guided_choice_token_ids)
            if done and not longer:
                return RequestStatus.FINISHED_STOPPED, None      # the chosen string is complete
        if (sp.max_tokens is not None and n_out >= sp.max_tokens) or req.num_tokens >= self.config.max_model_len:
            return RequestStatus.FINISHED_LENGTH, None
        return None

    def _check_stop(self, req: Request) -> None:
        stop = self._stop_decision(req)
        if stop is not None:
            self._stop_running(req, *stop)

    def finish_request(self, req: Request, status: RequestStatus, stop_reason=None) -> None:
        """Used by the front end for stop strings detected after detokenisation."""
        if not req.status.finished:
            self._stop_running(req, status, stop_reason)

    def _stop_running(self, req: Request, status: RequestStatus, stop_reason) -> None:
        if req in self.running:
            self.running.remove(req)
        req.stop_reason = stop_reason
        self._finish(req, status)

    def _finish(self, req: Request, status: RequestStatus) -> None:
        req.status = status
        req.finished_time = time.monotonic()
        self.kv.free(req)
        self._finished_since_last.append(req.request_id)
        self.requests.pop(req.request_id, None)
