"""Multi-process executor: the engine process spawns one worker process per GPU, broadcasts every RPC
through a shared-memory message queue and collects one response per worker.

Counterpart of vllm/v1/executor/multiproc_executor.py:44-481: readiness handshake, a monitor thread on
the workers' process sentinels (a dead worker marks the executor failed and fires the failure
callback), per-call timeouts (30 s for ``execute_model``, 180 s otherwise), exceptions in a worker
returned as FAILURE, and SIGTERM -> SIGKILL escalation at shutdown (only on the PIDs spawned here).
"""
from __future__ import annotations

import multiprocessing as mp
import os
import signal
import threading
import time
import traceback
from multiprocessing.connection import wait as mp_wait
from typing import Any, Optional

from .. import envs
from ..config import EngineConfig
from ..parallel.shm_broadcast import MessageQueue
from ..utils.logging import init_logger, set_process_prefix
from ..worker.model_runner import StepData, StepResult
from .base import Executor, ExecutorFailure

logger = init_logger(__name__)
_SHUTDOWN = "__shutdown__"


def _worker_main(config: EngineConfig, rank: int, init_method: str, mq_handle: tuple, resp_conn, ready_conn) -> None:
    set_process_prefix(f"(Worker_TP{rank} pid={os.getpid()})")
    signal.signal(signal.SIGINT, signal.SIG_IGN)
    worker = None
    try:
        from ..worker.worker import Worker
        mq = MessageQueue.attach(mq_handle, rank)
        worker = Worker(config, rank, config.parallel.device_offset + rank, init_method)
        worker.init_device()
        worker.load_model()
        ready_conn.send(("READY", rank))
    except Exception:
        ready_conn.send(("FAILED", traceback.format_exc()))
        return
    parent = os.getppid()
    # Host-side fault injection for tests. Honoured by CPU workers only: a GPU rank that exits while its
    # symmetric buffer is bound to an NVLink multicast object can fault its peers' GPUs.
    fail_at = exit_at = -1
    if worker.device.type == "cpu":
        fail_at = int(os.environ.get("TW_TEST_FAIL_AT_STEP", "-1"))
        exit_at = int(os.environ.get("TW_TEST_EXIT_AT_STEP", "-1"))
    fault_rank = int(os.environ.get("TW_TEST_FAULT_RANK", "0"))
    steps = 0
    while True:
        try:
            msg = mq.dequeue(timeout=None, should_stop=lambda: os.getppid() != parent)
        except ConnectionError:
            break
        if msg == _SHUTDOWN:
            break
        method, args, kwargs = msg
        try:
            if method == "execute_model":
                steps += 1
                if rank == fault_rank and steps == exit_at:
                    os._exit(17)                      # a rank that dies between steps
                if rank == fault_rank and steps == fail_at:
                    raise RuntimeError("injected failure in execute_model")
            result = getattr(worker, method)(*args, **kwargs)
            resp_conn.send(("SUCCESS", result))
        except Exception as e:
            resp_conn.send(("FAILURE", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    try:
        worker.shutdown()
    except Exception:
        pass


class MultiprocExecutor(Executor):
    def __init__(self, config: EngineConfig):
        super().__init__(config)
        self.world = config.parallel.world_size
        ctx = mp.get_context(envs.TW_WORKER_MULTIPROC_METHOD)
        from ..parallel.state import TPState  # noqa: F401  (import check before spawning)
        import socket
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        init_method = f"tcp://127.0.0.1:{port}"
        self.mq = MessageQueue.create(self.world)
        self.procs, self.resp, readies = [], [], []
        self._shutting_down = False
        for rank in range(self.world):
            resp_r, resp_w = ctx.Pipe(duplex=False)
            ready_r, ready_w = ctx.Pipe(duplex=False)
            p = ctx.Process(target=_worker_main, args=(config, rank, init_method, self.mq.handle(), resp_w, ready_w),
                            name=f"tw-worker-{rank}", daemon=True)
            p.start()
            resp_w.close()
            ready_w.close()
            self.procs.append(p)
            self.resp.append(resp_r)
            readies.append(ready_r)
        deadline = time.monotonic() + 600
        for rank, conn in enumerate(readies):
            if not conn.poll(max(0.0, deadline - time.monotonic())):
                self.shutdown()
                raise ExecutorFailure(f"worker {rank} did not become ready")
            try:
                status, info = conn.recv()
            except EOFError:
                self.shutdown()
                raise ExecutorFailure(f"worker {rank} died during start-up")
            if status != "READY":
                self.shutdown()
                raise ExecutorFailure(f"worker {rank} failed to start:\n{info}")
        self._monitor = threading.Thread(target=self._monitor_workers, name="tw-worker-monitor", daemon=True)
        self._monitor.start()

    # ---- liveness ----
    def _monitor_workers(self) -> None:
        sentinels = [p.sentinel for p in self.procs]
        died = mp_wait(sentinels)
        if self._shutting_down:
            return
        dead = [p.name for p in self.procs if p.sentinel in died]
        logger.error("worker process(es) %s died unexpectedly", dead)
        self.is_failed = True
        if self.failure_callback is not None:
            self.failure_callback()

    def _alive(self) -> bool:
        return not self.is_failed and all(p.is_alive() for p in self.procs)

    # ---- RPC ----
    def collective_rpc(self, method: str, *args, timeout: Optional[float] = None, **kwargs) -> list[Any]:
        if self.is_failed:
            raise ExecutorFailure("executor has failed")
        timeout = envs.TW_RPC_TIMEOUT_S if timeout is None else timeout
        try:
            self.mq.enqueue((method, args, kwargs), timeout=timeout, should_stop=lambda: not self._alive())
        except (TimeoutError, ConnectionError) as e:
            self.is_failed = True
            raise ExecutorFailure(f"could not deliver {method}: {e}") from e
        results = []
        deadline = time.monotonic() + timeout
        for rank, conn in enumerate(self.resp):
            while True:
                left = deadline - time.monotonic()
                if left <= 0:
                    self.is_failed = True
                    raise ExecutorFailure(f"worker {rank} did not answer {method} within {timeout:.0f}s")
                if conn.poll(min(left, 0.2)):
                    try:
                        status, payload = conn.recv()
                    except EOFError:
                        self.is_failed = True
                        raise ExecutorFailure(f"worker {rank} died while running {method}")
                    break
                if not self.procs[rank].is_alive():
                    self.is_failed = True
                    raise ExecutorFailure(f"worker {rank} died while running {method}")
            if status != "SUCCESS":
                self.is_failed = True
                raise ExecutorFailure(f"worker {rank} failed in {method}: {payload}")
            results.append(payload)
        return results

    def determine_num_blocks(self) -> int:
        return min(self.collective_rpc("determine_num_blocks"))

    def init_kv_cache(self, num_blocks: int) -> None:
        self.collective_rpc("init_kv_cache", num_blocks)

    def execute_model(self, step: StepData) -> StepResult:
        return self.collective_rpc("execute_model", step, timeout=envs.TW_EXECUTE_MODEL_TIMEOUT_S)[0]

    def shutdown(self) -> None:
        if self._shutting_down:
            return
        self._shutting_down = True
        try:
            if all(p.is_alive() for p in self.procs):
                self.mq.enqueue(_SHUTDOWN, timeout=2.0)
        except Exception:
            pass
        deadline = time.monotonic() + 5
        for p in self.procs:
            p.join(max(0.0, deadline - time.monotonic()))
        for p in self.procs:
            if p.is_alive():
                p.terminate()                      # SIGTERM to this child's PID only
        for p in self.procs:
            p.join(2)
            if p.is_alive():
                p.kill()                           # SIGKILL escalation
                p.join(1)
        for c in self.resp:
            try:
                c.close()
            except Exception:
                pass
        self.mq.close()
