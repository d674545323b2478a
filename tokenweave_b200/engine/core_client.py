"""Engine core in a process of its own, behind ZMQ sockets and msgpack.

Counterpart of vllm/v1/engine/core.py:346-407 (``EngineCoreProc.run_engine_core`` / ``run_busy_loop``) and
vllm/v1/engine/core_client.py:472-545 (``SyncMPClient``). With ``engine_core_process=True`` the scheduler, the
KV-block manager and the executor leave the front-end process: tokenisation, detokenisation, stop strings and
output assembly then run concurrently with the next step's scheduling and kernel launches instead of sharing
one Python thread with them.

Wire format: every message is one msgpack map ``{"t": type, ...}``; requests go core-wards over a PUSH/PULL
pair, step results come back over a second one (``ipc://`` endpoints in a private temporary directory).

* front end -> core: ``add`` (a request: ids, sampling parameters as a map, adapter, priority), ``abort``,
  ``finish`` (a stop string matched after detokenisation), ``rpc`` (``collective_rpc`` on the executor),
  ``shutdown``;
* core -> front end: ``ready`` (block count) or ``failed`` once at start-up, ``step`` (per touched request:
  new tokens, status, stop reason, log-probabilities, prompt log-probabilities, pooled vector, timestamps;
  plus the step statistics), ``rpc_result``, ``dead`` (the engine cannot go on; the reason).

The front end keeps a mirror :class:`~tokenweave_b200.engine.request.Request` per request, updated from the
``step`` messages, so :class:`~tokenweave_b200.engine.llm_engine.LLMEngine` works on either kind of core.
The core steps whenever it has unfinished requests (a busy loop): results queue up on the socket and
``step()`` on this side hands them out one engine step at a time.
"""
from __future__ import annotations

import dataclasses
import multiprocessing as mp
import os
import shutil
import tempfile
import time
import traceback
from typing import Optional

import msgpack
import zmq

from ..config import EngineConfig
from ..sampling_params import SamplingParams
from ..utils.logging import init_logger
from ..utils.metrics import StepStats
from .core import EngineCore, EngineDeadError
from .request import Request, RequestStatus

logger = init_logger(__name__)

_STARTUP_TIMEOUT_S = 900.0


# ---- encoding ------------------------------------------------------------------------------------
def _pack(obj: dict) -> bytes:
    return msgpack.packb(obj, use_bin_type=True)


def _unpack(raw: bytes) -> dict:
    return msgpack.unpackb(raw, raw=False, strict_map_key=False)


def encode_request(req: Request) -> dict:
    lora = None
    if req.lora_request is not None:
        lora = dataclasses.asdict(req.lora_request)
    return {"t": "add", "id": req.request_id, "ids": list(req.prompt_token_ids),
            "sp": dataclasses.asdict(req.sampling_params), "eos": req.eos_token_id, "prompt": req.prompt,
            "lora": lora, "prio": req.priority}


def decode_request(msg: dict) -> Request:
    lora = None
    if msg.get("lora") is not None:
        from ..lora import LoRARequest
        lora = LoRARequest(**msg["lora"])
    return Request(msg["id"], list(msg["ids"]), SamplingParams(**msg["sp"]), eos_token_id=msg.get("eos"),
                   prompt=msg.get("prompt"), lora_request=lora, priority=msg.get("prio", 0))


def _encode_touched(req: Request, sent: dict, logprob) -> dict:
    """What changed for one request in a step: the tokens beyond those already sent, and its state."""
    n = sent.get(req.request_id, 0)
    new = req.output_token_ids[n:]
    sent[req.request_id] = len(req.output_token_ids)
    out = {"id": req.request_id, "new": list(new), "st": int(req.status), "stop": req.stop_reason,
           "t_sched": req.first_scheduled_time, "t_first": req.first_token_time, "t_fin": req.finished_time}
    if logprob is not None:
        out["lp"] = {int(k): float(v) for k, v in logprob.items()}
    if req.prompt_logprobs:
        out["plp"] = {int(p): {int(k): float(v) for k, v in d.items()} for p, d in req.prompt_logprobs.items()}
    if req.pooled is not None:
        out["pooled"] = [float(x) for x in req.pooled.tolist()]
    return out


# ---- the core process -------------------------------------------------------------------------------
def _core_main(config: EngineConfig, in_addr: str, out_addr: str) -> None:
    ctx = zmq.Context()
    inp = ctx.socket(zmq.PULL)
    inp.connect(in_addr)
    out = ctx.socket(zmq.PUSH)
    out.connect(out_addr)
    try:
        core = EngineCore(config)
    except Exception:
        out.send(_pack({"t": "failed", "why": traceback.format_exc()}))
        return
    out.send(_pack({"t": "ready", "num_blocks": core.num_blocks}))
    sent: dict[str, int] = {}
    parent = os.getppid()
    try:
        while True:
            # block for input only when there is nothing to run
            if os.getppid() != parent:
                break                              # the front end is gone
            busy = core.has_unfinished_requests()
            if not busy and not inp.poll(1000):
                continue
            stop = False
            while inp.poll(0):
                msg = _unpack(inp.recv())
                t = msg["t"]
                if t == "add":
                    try:
                        core.add_request(decode_request(msg))
                    except Exception as e:          # a bad request must not take the engine down
                        out.send(_pack({"t": "rejected", "id": msg["id"], "why": f"{type(e).__name__}: {e}"}))
                elif t == "abort":
                    core.abort_request(msg["id"])
                    sent.pop(msg["id"], None)
                elif t == "finish":
                    req = core.scheduler.requests.get(msg["id"])
                    if req is not None:
                        core.scheduler.finish_request(req, RequestStatus(msg["st"]), msg.get("stop"))
                    sent.pop(msg["id"], None)
                elif t == "rpc":
                    try:
                        if msg.get("core"):         # a call on the core itself, not on the workers
                            if msg["name"] != "reset_prefix_cache":
                                raise ValueError(f"unknown core call {msg['name']!r}")
                            res = core.scheduler.kv.pool.reset_prefix_cache()
                        else:
                            res = core.executor.collective_rpc(msg["name"], *msg.get("args", []))
                        out.send(_pack({"t": "rpc_result", "ok": True, "res": _plain(res)}))
                    except Exception as e:
                        out.send(_pack({"t": "rpc_result", "ok": False, "res": f"{type(e).__name__}: {e}"}))
                elif t == "shutdown":
                    stop = True
            if stop:
                break
            if core.has_unfinished_requests():
                touched = core.step()
                lps = getattr(core, "_last_logprobs", {})
                items = [_encode_touched(r, sent, lps.get(r.request_id)) for r in touched]
                for r in touched:
                    if r.status.finished:
                        sent.pop(r.request_id, None)
                stats = dataclasses.asdict(core.last_stats) if core.last_stats is not None else None
                out.send(_pack({"t": "step", "items": items, "stats": stats,
                                "unfinished": core.scheduler.num_unfinished()}))
    except Exception:
        out.send(_pack({"t": "dead", "why": traceback.format_exc()}))
    finally:
        try:
            core.shutdown()
        except Exception:
            pass
        inp.close(0)
        out.close(1000)
        ctx.term()


def _plain(x):
    """RPC results cross the socket as plain msgpack values (anything else by its ``repr``)."""
    if x is None or isinstance(x, (bool, int, float, str, bytes)):
        return x
    if isinstance(x, (list, tuple)):
        return [_plain(v) for v in x]
    if isinstance(x, dict):
        return {str(k): _plain(v) for k, v in x.items()}
    return repr(x)


# ---- the front-end side -----------------------------------------------------------------------------
class _SchedulerProxy:
    """The two scheduler calls the front end makes, forwarded to the core process."""

    def __init__(self, client: "MPEngineCoreClient"):
        self._c = client
        self.requests = client.mirror

    def num_unfinished(self) -> int:
        return len(self._c.mirror)

    def finish_request(self, req: Request, status: RequestStatus, stop_reason=None) -> None:
        if req.status.finished:
            return
        req.status, req.stop_reason, req.finished_time = status, stop_reason, time.monotonic()
        self._c.mirror.pop(req.request_id, None)
        self._c._send({"t": "finish", "id": req.request_id, "st": int(status), "stop": stop_reason})


class _ExecutorProxy:
    def __init__(self, client: "MPEngineCoreClient"):
        self._c = client

    def collective_rpc(self, name: str, *args):
        return self._c.rpc(name, *args)


class MPEngineCoreClient:
    """Same surface as :class:`EngineCore` for the front end; the core itself runs in a child process."""

    def __init__(self, config: EngineConfig):
        self.config = config
        self.dead = False
        self.mirror: dict[str, Request] = {}
        self.last_stats: Optional[StepStats] = None
        self._last_logprobs: dict = {}
        self._dir = tempfile.mkdtemp(prefix="tw_core_")
        in_addr, out_addr = f"ipc://{self._dir}/in", f"ipc://{self._dir}/out"
        self._ctx = zmq.Context()
        self._to_core = self._ctx.socket(zmq.PUSH)
        self._to_core.bind(in_addr)
        self._from_core = self._ctx.socket(zmq.PULL)
        self._from_core.bind(out_addr)
        self._proc = mp.get_context("spawn").Process(target=_core_main, args=(config, in_addr, out_addr),
                                                     name="tw-engine-core", daemon=False)
        self._proc.start()
        msg = self._recv(_STARTUP_TIMEOUT_S)
        if msg["t"] != "ready":
            self.shutdown()
            raise RuntimeError(f"engine core did not start:\n{msg.get('why', msg)}")
        self.num_blocks = msg["num_blocks"]
        self.scheduler = _SchedulerProxy(self)
        self.executor = _ExecutorProxy(self)

    # ---- plumbing ----
    def _send(self, msg: dict) -> None:
        if self.dead:
            raise EngineDeadError("engine core is dead")
        data = _pack(msg)
        deadline = time.monotonic() + self.config.engine_core_timeout_s
        while True:
            # a PUSH socket whose peer is gone blocks in send(): poll for room and watch the process instead
            if not self._proc.is_alive():
                self.dead = True
                raise EngineDeadError(f"engine core process exited with code {self._proc.exitcode}")
            if self._to_core.poll(200, zmq.POLLOUT):
                self._to_core.send(data, zmq.NOBLOCK)
                return
            if time.monotonic() > deadline:
                self.dead = True
                raise EngineDeadError("engine core process does not take requests")

    def _recv(self, timeout_s: float) -> dict:
        deadline = time.monotonic() + timeout_s
        while True:
            if self._from_core.poll(200):
                return _unpack(self._from_core.recv())
            if not self._proc.is_alive():
                self.dead = True
                raise EngineDeadError(f"engine core process exited with code {self._proc.exitcode}")
            if time.monotonic() > deadline:
                self.dead = True
                raise EngineDeadError("engine core process does not answer")

    # ---- EngineCore surface ----
    def add_request(self, req: Request) -> None:
        self._send(encode_request(req))
        self.mirror[req.request_id] = req

    def abort_request(self, request_id: str) -> None:
        req = self.mirror.pop(request_id, None)
        if req is not None and not req.status.finished:
            req.status, req.finished_time = RequestStatus.FINISHED_ABORTED, time.monotonic()
            self._send({"t": "abort", "id": request_id})

    def has_unfinished_requests(self) -> bool:
        return bool(self.mirror)

    def step(self) -> list[Request]:
        """The next engine step's results (blocks until the core has produced them)."""
        if self.dead:
            raise EngineDeadError("engine core is dead")
        if not self.mirror:
            return []
        while True:
            msg = self._recv(self.config.engine_core_timeout_s)
            t = msg["t"]
            if t == "step":
                return self._apply_step(msg)
            if t == "rejected":
                req = self.mirror.pop(msg["id"], None)
                if req is not None:
                    req.status, req.finished_time = RequestStatus.FINISHED_ABORTED, time.monotonic()
                    req.stop_reason = msg["why"]
                    return [req]
                continue
            if t == "dead":
                self.dead = True
                raise EngineDeadError(msg.get("why", "engine core failed"))
            # anything else (a late rpc_result) is dropped

    def _apply_step(self, msg: dict) -> list[Request]:
        touched = []
        self._last_logprobs = {}
        for it in msg["items"]:
            req = self.mirror.get(it["id"])
            if req is None or req.status.finished:
                continue              # aborted or stopped on this side while the core was a step ahead
            req.output_token_ids.extend(it["new"])
            req.status = RequestStatus(it["st"])
            req.stop_reason = it.get("stop")
            req.first_scheduled_time = it.get("t_sched") or req.first_scheduled_time
            req.first_token_time = it.get("t_first") or req.first_token_time
            req.finished_time = it.get("t_fin")
            if "lp" in it:
                self._last_logprobs[req.request_id] = it["lp"]
            if "plp" in it:
                req.prompt_logprobs.update(it["plp"])
            if "pooled" in it and req.pooled is None:
                import torch
                req.pooled = torch.tensor(it["pooled"], dtype=torch.float32)
            if req.status.finished:
                self.mirror.pop(req.request_id, None)
            touched.append(req)
        self.last_stats = StepStats(**msg["stats"]) if msg.get("stats") else None
        return touched

    def rpc_core(self, name: str):
        return self.rpc(name, on_core=True)

    def rpc(self, name: str, *args, on_core: bool = False):
        if self.mirror:
            raise RuntimeError("collective_rpc needs an idle engine when the core runs in its own process")
        self._send({"t": "rpc", "name": name, "args": list(args), "core": on_core})
        while True:
            msg = self._recv(self.config.engine_core_timeout_s)
            if msg["t"] == "rpc_result":
                if not msg["ok"]:
                    raise RuntimeError(msg["res"])
                return msg["res"]
            if msg["t"] == "dead":
                self.dead = True
                raise EngineDeadError(msg.get("why", "engine core failed"))

    def shutdown(self) -> None:
        if getattr(self, "_proc", None) is None:
            return
        try:
            if self._proc.is_alive() and self._to_core.poll(1000, zmq.POLLOUT):
                self._to_core.send(_pack({"t": "shutdown"}), zmq.NOBLOCK)
                self._proc.join(30)
            if self._proc.is_alive():
                self._proc.terminate()
                self._proc.join(10)
        finally:
            self._to_core.close(0)
            self._from_core.close(0)
            self._ctx.term()
            shutil.rmtree(self._dir, ignore_errors=True)
            self._proc = None
