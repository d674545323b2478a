"""Executor interface (counterpart of vllm/v1/executor/abstract.py:56-112)."""
from __future__ import annotations

from typing import Any, Callable, Optional

from ..config import EngineConfig
from ..worker.model_runner import StepData, StepResult


class ExecutorFailure(RuntimeError):
    """A worker died, raised, or did not answer in time."""


class Executor:
    def __init__(self, config: EngineConfig):
        self.config = config
        self.failure_callback: Optional[Callable[[], None]] = None
        self.is_failed = False

    def determine_num_blocks(self) -> int:
        raise NotImplementedError

    def init_kv_cache(self, num_blocks: int) -> None:
        raise NotImplementedError

    def execute_model(self, step: StepData) -> StepResult:
        raise NotImplementedError

    def collective_rpc(self, method: str, *args, timeout: Optional[float] = None, **kwargs) -> list[Any]:
        raise NotImplementedError

    def profile(self, start: bool) -> None:
        self.collective_rpc("profile", start)

    def check_health(self) -> None:
        self.collective_rpc("check_health")

    def register_failure_callback(self, cb: Callable[[], None]) -> None:
        self.failure_callback = cb

    def shutdown(self) -> None:
        pass


def make_executor(config: EngineConfig) -> Executor:
    import os
    backend = config.parallel.distributed_executor_backend
    tp = config.parallel.world_size          # ranks of the replica: tensor-parallel x pipeline-parallel
    if backend == "auto":
        if tp == 1:
            backend = "uni"
        elif int(os.environ.get("WORLD_SIZE", "1")) == tp and "RANK" in os.environ:
            backend = "external_launcher"
        else:
            backend = "mp"
    if backend in ("uni", "external_launcher"):
        from .uniproc import UniProcExecutor
        return UniProcExecutor(config, external_launcher=(backend == "external_launcher"))
    if backend == "mp":
        from .multiproc import MultiprocExecutor
        return MultiprocExecutor(config)
    raise ValueError(f"unknown distributed_executor_backend {backend!r}")
