"""In-process executor. With ``external_launcher`` the process is one rank of a ``torchrun`` job:
every rank runs the same engine on the same request stream (the scheduler is deterministic), so the
ranks meet in the collectives of the model without any control messages
(counterpart of the reference's ExecutorWithExternalLauncher, vllm/executor/uniproc_executor.py)."""
from __future__ import annotations

import os
from typing import Any, Optional

from ..config import EngineConfig
from ..worker.model_runner import StepData, StepResult
from ..worker.worker import Worker
from .base import Executor


class UniProcExecutor(Executor):
    def __init__(self, config: EngineConfig, external_launcher: bool = False):
        super().__init__(config)
        if external_launcher:
            rank = int(os.environ.get("RANK", "0"))
            local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
            world = int(os.environ.get("WORLD_SIZE", "1"))
            if world != config.parallel.world_size:
                raise ValueError(f"WORLD_SIZE={world} does not match tensor_parallel_size x pipeline_parallel_size="
                                 f"{config.parallel.world_size}")
        else:
            if config.parallel.world_size != 1:
                raise ValueError("the in-process executor runs one rank; use the 'mp' or "
                                 "'external_launcher' backend for tensor or pipeline parallelism")
            rank, local_rank = 0, config.parallel.device_offset
        self.rank = rank
        self.worker = Worker(config, rank, local_rank)
        self.worker.init_device()
        self.worker.load_model()

    def determine_num_blocks(self) -> int:
        n = self.worker.determine_num_blocks()
        if self.config.parallel.world_size > 1:
            import torch
            import torch.distributed as dist
            from ..parallel.state import get_tp
            t = torch.tensor([n], dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=get_tp().world_cpu_group)       # all stages agree
            n = int(t.item())
        return n

    def init_kv_cache(self, num_blocks: int) -> None:
        self.worker.init_kv_cache(num_blocks)

    def execute_model(self, step: StepData) -> StepResult:
        return self.worker.execute_model(step)

    def collective_rpc(self, method: str, *args, timeout: Optional[float] = None, **kwargs) -> list[Any]:
        return [getattr(self.worker, method)(*args, **kwargs)]

    def shutdown(self) -> None:
        if self.worker is not None:
            self.worker.shutdown()
            self.worker = None
