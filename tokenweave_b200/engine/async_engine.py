"""Asynchronous front of the engine for online serving: one background thread owns the ``LLMEngine``
and steps it while requests are in flight; callers on an asyncio loop add requests and receive
``RequestOutput`` snapshots through per-request queues.

Counterpart of vllm/v1/engine/async_llm.py (``AsyncLLM.generate`` / ``abort`` / the output-handler
loop). The reference moves the engine core into its own process and talks to it over ZMQ
(vllm/v1/engine/core_client.py); here the core stays in-process — the GPU work is asynchronous to
the host anyway — and only the request hand-off crosses threads.
"""
from __future__ import annotations

import asyncio
import queue
import threading
from typing import AsyncIterator, Optional, Union

from ..config import EngineArgs
from ..outputs import RequestOutput
from ..sampling_params import SamplingParams
from ..utils.logging import init_logger
from .llm_engine import LLMEngine

logger = init_logger(__name__)


class EngineDeadError(RuntimeError):
    """The engine loop stopped on an exception; no further request can be served."""


class AsyncLLMEngine:
    def __init__(self, engine: LLMEngine):
        self.engine = engine
        self._inbox: "queue.Queue[tuple]" = queue.Queue()
        self._streams: dict[str, tuple[asyncio.AbstractEventLoop, asyncio.Queue]] = {}
        self._lock = threading.Lock()
        self._wake = threading.Event()
        self._stop = False
        self._dead: Optional[BaseException] = None
        self._thread = threading.Thread(target=self._loop, name="tw-engine-loop", daemon=True)
        self._thread.start()

    @classmethod
    def from_engine_args(cls, args: EngineArgs) -> "AsyncLLMEngine":
        return cls(LLMEngine.from_engine_args(args))

    # ---- engine thread ------------------------------------------------------------------------
    def _deliver(self, rid: str, item) -> None:
        with self._lock:
            target = self._streams.get(rid)
        if target is None:
            return
        loop, q = target
        loop.call_soon_threadsafe(q.put_nowait, item)

    def _loop(self) -> None:
        try:
            while not self._stop:
                drained = False
                while True:
                    try:
                        kind, rid, prompt, params, lora = self._inbox.get_nowait()
                    except queue.Empty:
                        break
                    drained = True
                    if kind == "add":
                        try:
                            self.engine.add_request(rid, prompt, params, lora_request=lora)
                        except Exception as e:      # bad request: report to its caller, keep serving
                            self._deliver(rid, e)
                    else:
                        self.engine.abort_request(rid)
                if self.engine.has_unfinished_requests():
                    for out in self.engine.step():
                        self._deliver(out.request_id, out)
                elif not drained:
                    self._wake.wait(timeout=0.05)
                    self._wake.clear()
        except BaseException as e:    # noqa: BLE001 - reported to every waiting caller
            logger.exception("engine loop died")
            self._dead = e
            with self._lock:
                targets = list(self._streams.items())
            for rid, (loop, q) in targets:
                loop.call_soon_threadsafe(q.put_nowait, EngineDeadError(str(e)))

    # ---- asyncio side -------------------------------------------------------------------------
    @property
    def is_running(self) -> bool:
        return self._thread.is_alive() and self._dead is None

    async def generate(self, prompt: Union[str, list[int], dict], params: SamplingParams,
                       request_id: str, lora_request=None) -> AsyncIterator[RequestOutput]:
        """Yields a snapshot of the request after every engine step that touched it; the last one has
        ``finished`` set. Cancelling the consumer aborts the request."""
        if self._dead is not None:
            raise EngineDeadError(str(self._dead))
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        with self._lock:
            if request_id in self._streams:
                raise ValueError(f"request id {request_id} is already in flight")
            self._streams[request_id] = (loop, q)
        self._inbox.put(("add", request_id, prompt, params, lora_request))
        self._wake.set()
        finished = False
        try:
            while True:
                item = await q.get()
                if isinstance(item, BaseException):
                    finished = True
                    raise item
                yield item
                if item.finished:
                    finished = True
                    return
        finally:
            with self._lock:
                self._streams.pop(request_id, None)
            if not finished:
                self._inbox.put(("abort", request_id, None, None, None))
                self._wake.set()

    async def abort(self, request_id: str) -> None:
        self._inbox.put(("abort", request_id, None, None, None))
        self._wake.set()

    def shutdown(self) -> None:
        self._stop = True
        self._wake.set()
        self._thread.join(timeout=10)
        self.engine.shutdown()
