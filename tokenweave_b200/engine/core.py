"""Engine core: schedule -> execute -> update, once per step.

Counterpart of vllm/v1/engine/core.py:47-249. The reference runs the core in a process of its own and
talks to it over ZMQ; here it runs in the caller's process (the executor below it is where process
boundaries are), which removes one serialisation hop from every step.
"""
from __future__ import annotations

from typing import Optional

from ..config import EngineConfig
from ..executor import Executor, make_executor
from ..executor.base import ExecutorFailure
from ..ops import KernelStatusError
from ..utils.logging import init_logger
from ..utils.metrics import StepStats
from ..worker.model_runner import NewRequestData, StepData, StepResult
from .kv_cache import KVCacheManager
from .request import Request
from .scheduler import ModelRunnerOutput, Scheduler, SchedulerOutput

logger = init_logger(__name__)


class EngineDeadError(RuntimeError):
    """The executor failed; the engine cannot make progress (vllm/v1/engine/exceptions.py)."""


class EngineCore:
    def __init__(self, config: EngineConfig, executor: Optional[Executor] = None):
        self.config = config
        self.executor = executor or make_executor(config)
        self.executor.register_failure_callback(self._on_executor_failure)
        self.dead = False
        num_blocks = self.executor.determine_num_blocks()
        self.executor.init_kv_cache(num_blocks)
        self.num_blocks = num_blocks
        self.kv = KVCacheManager(num_blocks, config.cache.block_size, config.cache.enable_prefix_caching)
        self.scheduler = Scheduler(config.scheduler, self.kv, config.speculative)
        self._sent_blocks: dict[str, int] = {}     # blocks of each request already known to the workers
        # KV connector: the scheduler side only asks which blocks the store can supply; the workers move the data
        self.kv_transfer = config.kv_transfer
        if self.kv_transfer is not None:
            from .kv_connector import kv_fingerprint, make_connector
            lookup = make_connector(self.kv_transfer, 0, config.parallel.world_size, kv_fingerprint(config),
                                    host_store=True)
            self.kv.track_published = self.kv_transfer.can_save
            if self.kv_transfer.can_load:
                self.scheduler.connector = lookup
        self.last_stats: Optional[StepStats] = None

    def _on_executor_failure(self) -> None:
        self.dead = True

    def add_request(self, req: Request) -> None:
        if self.dead:
            raise EngineDeadError("engine core is dead")
        self.scheduler.add_request(req)

    def abort_request(self, request_id: str) -> None:
        self.scheduler.abort_request(request_id)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished_requests()

    def _to_step_data(self, out: SchedulerOutput) -> StepData:
        step = StepData(step_id=out.step_id, finished_req_ids=list(out.finished_req_ids),
                        preempted_req_ids=list(out.preempted_req_ids), total_num_tokens=out.total_num_tokens)
        for rid in out.finished_req_ids + out.preempted_req_ids:
            self._sent_blocks.pop(rid, None)
        for s in out.scheduled:
            r = s.request
            if s.is_new:
                step.new_requests.append(NewRequestData(r.request_id, r.all_token_ids, r.num_prompt_tokens,
                                                        r.sampling_params, list(r.block_ids), r.lora_request))
                new_blocks: list[int] = []
            else:
                new_blocks = r.block_ids[self._sent_blocks.get(r.request_id, 0):]
            self._sent_blocks[r.request_id] = len(r.block_ids)
            step.scheduled.append((r.request_id, s.num_computed_tokens, s.num_new_tokens, list(new_blocks),
                                   list(s.spec_token_ids)))
        return step

    def step(self) -> list[Request]:
        """One engine iteration. Returns the requests that produced a token or finished."""
        if self.dead:
            raise EngineDeadError("engine core is dead")
        sched = self.scheduler.schedule()
        if sched.empty:
            if sched.finished_req_ids:
                # let the workers drop finished requests even when nothing is scheduled
                self.executor.execute_model(self._to_step_data(sched))
            return []
        try:
            if sched.kv_loads:
                self.executor.collective_rpc("load_kv_blocks", list(sched.kv_loads))
            result: StepResult = self.executor.execute_model(self._to_step_data(sched))
        except ExecutorFailure as e:
            self.dead = True
            raise EngineDeadError(str(e)) from e
        except KernelStatusError as e:
            # an in-process worker read a non-zero device status word with the step's result: the collectives
            # of this step did not complete, nothing of it is emitted, and the signal pads / tile flags are in an
            # unknown state until the workers run ``reset_comm_state`` together
            self.dead = True
            raise EngineDeadError(f"a kernel reported a failed wait: {e}") from e
        if result.prompt_logprobs:
            by_id = {s.request.request_id: s.request for s in sched.scheduled}
            for rid, items in result.prompt_logprobs.items():
                if rid in by_id:
                    by_id[rid].prompt_logprobs.update(items)      # keyed by position: a recompute overwrites
        if result.pooled:
            for s in sched.scheduled:
                vec = result.pooled.get(s.request.request_id)
                if vec is not None and s.request.pooled is None:
                    s.request.pooled = vec
        touched = self.scheduler.update_from_output(
            sched, ModelRunnerOutput(result.req_ids, result.sampled_token_ids, result.logprobs))
        self._last_logprobs = dict(zip(result.req_ids, result.logprobs)) if result.logprobs else {}
        if self.kv.newly_published:
            # blocks that became full in this step are in the workers' caches now: publish them to the store
            saves, self.kv.newly_published = self.kv.newly_published, []
            try:
                self.executor.collective_rpc("save_kv_blocks", saves)
            except ExecutorFailure as e:
                self.dead = True
                raise EngineDeadError(str(e)) from e
        self.last_stats = StepStats(num_tokens=sched.total_num_tokens, num_running=len(self.scheduler.running),
                                    num_waiting=len(self.scheduler.waiting), kv_usage=self.kv.usage(),
                                    num_generated=self.scheduler.last_emitted,
                                    prefix_cache_queries=self.kv.prefix_queries, prefix_cache_hits=self.kv.prefix_hits,
                                    num_draft_tokens=self.scheduler.num_draft_tokens,
                                    num_accepted_tokens=self.scheduler.num_accepted_tokens)
        return touched

    def shutdown(self) -> None:
        if self.executor is not None:
            self.executor.shutdown()
            self.executor = None
