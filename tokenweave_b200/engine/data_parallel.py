"""Data parallelism for online serving: several independent engine replicas behind one front end.

Counterpart of the reference's data-parallel engine cores (vllm/v1/engine/core.py ``DPEngineCoreProc`` and
the load-balancing client in vllm/v1/engine/core_client.py): every replica is a complete engine — scheduler,
KV cache and a tensor-parallel worker group on its own GPUs (replica ``r`` owns devices
``[r * tp, (r + 1) * tp)``) — and a request is routed to the replica with the fewest requests in flight.
Dense models need no traffic between replicas; the reference's periodic "any replica unfinished" all-reduce
only exists to keep expert-parallel MoE layers in lock step across replicas, a layout that is not built here
(experts are sharded inside a replica's TP group).

On GPUs the replicas use the multi-process executor, so each replica's ranks live in their own processes and
process groups; the front process only holds the schedulers and the request queues.
"""
from __future__ import annotations

import dataclasses
import itertools
from typing import AsyncIterator, Union

from ..config import EngineArgs
from ..outputs import RequestOutput
from ..sampling_params import SamplingParams
from ..utils.logging import init_logger
from .async_engine import AsyncLLMEngine

logger = init_logger(__name__)


class DataParallelEngine:
    """Same surface as :class:`AsyncLLMEngine` (``generate`` / ``abort`` / ``is_running`` / ``shutdown`` and
    ``.engine`` for configuration and tokenizer access), backed by ``data_parallel_size`` replicas."""

    def __init__(self, replicas: list[AsyncLLMEngine]):
        if not replicas:
            raise ValueError("at least one replica")
        self.replicas = replicas
        self.in_flight = [0] * len(replicas)
        self.served = [0] * len(replicas)          # requests routed to each replica so far
        self._where: dict[str, int] = {}
        self._rr = itertools.count()

    @classmethod
    def from_engine_args(cls, args: EngineArgs) -> "DataParallelEngine":
        import torch
        n = args.data_parallel_size
        on_gpu = args.device == "cuda" or (args.device == "auto" and torch.cuda.is_available())
        replicas = []
        try:
            for r in range(n):
                a = dataclasses.replace(args, data_parallel_rank=r)
                if on_gpu and a.distributed_executor_backend in ("auto", "uni"):
                    a.distributed_executor_backend = "mp"      # one process group per replica
                logger.info("starting data-parallel replica %d of %d", r, n)
                replicas.append(AsyncLLMEngine.from_engine_args(a))
        except Exception:
            for e in replicas:
                e.shutdown()
            raise
        return cls(replicas)

    @property
    def engine(self):
        return self.replicas[0].engine

    @property
    def is_running(self) -> bool:
        return all(r.is_running for r in self.replicas)

    def _pick(self) -> int:
        alive = [i for i, r in enumerate(self.replicas) if r.is_running]
        if not alive:
            return 0                # generate() on a dead replica raises EngineDeadError for the caller
        low = min(self.in_flight[i] for i in alive)
        tied = [i for i in alive if self.in_flight[i] == low]
        return tied[next(self._rr) % len(tied)]

    async def generate(self, prompt: Union[str, list[int], dict], params: SamplingParams, request_id: str,
                       lora_request=None) -> AsyncIterator[RequestOutput]:
        i = self._pick()
        self.in_flight[i] += 1
        self.served[i] += 1
        self._where[request_id] = i
        try:
            async for out in self.replicas[i].generate(prompt, params, request_id, lora_request=lora_request):
                yield out
        finally:
            self.in_flight[i] -= 1
            self._where.pop(request_id, None)

    async def abort(self, request_id: str) -> None:
        i = self._where.get(request_id)
        if i is not None:
            await self.replicas[i].abort(request_id)

    def shutdown(self) -> None:
        for r in self.replicas:
            r.shutdown()
