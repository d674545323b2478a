"""OpenAI-compatible HTTP server on top of :class:`AsyncLLMEngine`.

    python -m tokenweave_b200.entrypoints.api_server --model <dir or preset> --tensor-parallel-size 1 --port 8000

Endpoints: ``GET /health``, ``GET /v1/models``, ``POST /v1/completions``, ``POST /v1/chat/completions``
(both with ``"stream": true`` server-sent events), ``POST /tokenize``, ``POST /detokenize``,
``GET /metrics`` (Prometheus text). A lean counterpart of vllm/entrypoints/openai/api_server.py and
serving_completion.py / serving_chat.py: the request fields that map onto ``SamplingParams`` are
honoured, including ``response_format`` and function calling (``tools`` / ``tool_choice``, entrypoints/tool_calls.py);
multimodal message parts are not served.
Tensor-parallel serving uses the multiprocess executor (one worker process per GPU).
"""
import argparse
import json
import os
import time
import uuid
from typing import Any, AsyncIterator, Optional

from ..config import EngineArgs
from ..engine.async_engine import AsyncLLMEngine, EngineDeadError
from ..outputs import RequestOutput
from ..sampling_params import SamplingParams
from ..utils.logging import init_logger

logger = init_logger(__name__)

_SAMPLING_FIELDS = ("n", "temperature", "top_p", "top_k", "min_p", "presence_penalty", "frequency_penalty",
                    "repetition_penalty", "seed", "stop", "stop_token_ids", "max_tokens", "min_tokens", "ignore_eos",
                    "skip_special_tokens", "logit_bias", "allowed_token_ids", "bad_words_token_ids", "guided_choice",
                    "prompt_logprobs", "guided_regex", "guided_json", "guided_grammar", "include_stop_str_in_output",
                    "truncate_prompt_tokens")


def sampling_params_from_request(body: dict, default_max_tokens: int = 16) -> SamplingParams:
    kw = {k: body[k] for k in _SAMPLING_FIELDS if body.get(k) is not None}
    # OpenAI's response_format: {"type": "json_object"} or {"type": "json_schema", "json_schema": {"schema": {...}}}
    rf = body.get("response_format")
    if isinstance(rf, dict) and "guided_json" not in kw and "guided_regex" not in kw:
        if rf.get("type") == "json_object":
            kw["guided_json"] = {}
        elif rf.get("type") == "json_schema":
            js = rf.get("json_schema") or {}
            kw["guided_json"] = js.get("schema", js)
    if "max_completion_tokens" in body and body["max_completion_tokens"] is not None:
        kw["max_tokens"] = body["max_completion_tokens"]
    kw.setdefault("max_tokens", default_max_tokens)
    lp = body.get("logprobs")
    if isinstance(lp, bool):            # chat schema: logprobs: true + top_logprobs: k
        lp = (body.get("top_logprobs") or 0) if lp else None
    if lp is not None:
        kw["logprobs"] = int(lp)
    return SamplingParams(**kw)


def _usage(out: RequestOutput) -> dict:
    gen = sum(len(c.token_ids) for c in out.outputs)
    return {"prompt_tokens": len(out.prompt_token_ids), "completion_tokens": gen,
            "total_tokens": len(out.prompt_token_ids) + gen}


def _logprobs_block(comp, tokenizer) -> Optional[dict]:
    if comp.logprobs is None:
        return None
    dec = (lambda t: tokenizer.decode([t])) if tokenizer is not None else (lambda t: str(t))
    toks = [dec(t) for t in comp.token_ids]
    chosen = [float(lp.get(t, 0.0)) for lp, t in zip(comp.logprobs, comp.token_ids)]
    top = [{dec(t): float(v) for t, v in lp.items()} for lp in comp.logprobs]
    return {"tokens": toks, "token_logprobs": chosen, "top_logprobs": top}


def build_app(engine: AsyncLLMEngine, served_model_name: Optional[str] = None,
              lora_modules: Optional[dict] = None, tool_call_parser: str = "auto",
              reasoning_parser: Optional[str] = None, api_key: Optional[str] = None,
              allowed_origins: Optional[list] = None):
    """``lora_modules`` maps a served adapter name to its directory: a request whose ``model`` field is
    such a name runs through that adapter (``--lora-modules name=path`` of the reference's server,
    vllm/entrypoints/openai/serving_models.py). ``tool_call_parser`` names the spelling of tool calls to look
    for in free text (entrypoints/tool_calls.py); ``reasoning_parser="deepseek_r1"`` moves ``<think>`` blocks of
    complete (non-streamed, or tool-calling) chat answers into ``reasoning_content``. ``api_key``: every ``/v1`` route
    then wants ``Authorization: Bearer <key>`` (``--api-key`` / the ``TW_API_KEY`` variable; the reference's
    vllm/entrypoints/openai/api_server.py authentication middleware); ``allowed_origins`` switches CORS headers on."""
    from .tool_calls import TOOL_CALL_PARSERS
    if tool_call_parser not in TOOL_CALL_PARSERS:
        raise ValueError(f"unknown tool-call parser {tool_call_parser!r}")
    if reasoning_parser not in (None, "deepseek_r1"):
        raise ValueError(f"unknown reasoning parser {reasoning_parser!r}")
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    from ..lora import LoRARequest

    app = FastAPI(title="tokenweave_b200")
    if allowed_origins:
        from fastapi.middleware.cors import CORSMiddleware
        app.add_middleware(CORSMiddleware, allow_origins=list(allowed_origins), allow_methods=["*"], allow_headers=["*"])
    if api_key:
        import hmac

        @app.middleware("http")
        async def authenticate(request: Request, call_next):
            if request.method != "OPTIONS" and request.url.path.startswith("/v1"):
                given = request.headers.get("Authorization", "")
                if not hmac.compare_digest(given.encode(), ("Bearer " + api_key).encode()):
                    return JSONResponse({"error": {"message": "invalid or missing API key", "type": "authentication_error",
                                                   "code": 401}}, status_code=401)
            return await call_next(request)
    model_cfg = engine.engine.config.model
    name = served_model_name or model_cfg.name
    tokenizer = engine.engine.tokenizer
    adapters = {n: LoRARequest(n, i + 1, path) for i, (n, path) in enumerate((lora_modules or {}).items())}

    def pick_adapter(body: dict):
        """The adapter a request names in ``model`` (None for the base model); unknown names are an error."""
        m = body.get("model")
        if m in adapters:
            return adapters[m]
        if m is None or not adapters or m == name or m == model_cfg.name:
            return None         # a server without adapters answers every model name with its one model
        raise ValueError(f"model {m!r} is not served (base model: {name!r}, adapters: {sorted(adapters)})")
    prom = None
    try:
        from ..utils.metrics import PrometheusStatLogger
        prom = PrometheusStatLogger(name)
        for e in getattr(engine, "replicas", [engine]):        # every data-parallel replica reports into it
            e.engine.stat_logger = prom
    except Exception:       # prometheus_client missing: /metrics answers 501
        prom = None

    def error(status: int, msg: str, typ: str = "invalid_request_error"):
        return JSONResponse({"error": {"message": msg, "type": typ, "code": status}}, status_code=status)

    def finished_metrics(out: RequestOutput) -> None:
        if prom is not None and out.finished:
            m = out.metrics
            n_out = max((len(c.token_ids) for c in out.outputs), default=0)
            tpot = ((m.finished_time - m.first_token_time) / (n_out - 1)
                    if m.finished_time and m.first_token_time and n_out > 1 else None)
            prom.record_finished((m.first_token_time - m.arrival_time) if m.first_token_time else None,
                                 (m.finished_time - m.arrival_time) if m.finished_time else None, tpot)

    @app.get("/health")
    async def health():
        return JSONResponse({"status": "ok"}) if engine.is_running else error(503, "engine is not running", "server_error")

    @app.get("/ping")
    async def ping():
        return await health()

    @app.get("/version")
    async def version():
        from .. import __version__
        return {"version": __version__}

    @app.get("/v1/models")
    async def models():
        card = lambda i, parent: {"id": i, "object": "model", "created": int(time.time()), "owned_by": "tokenweave_b200",  # noqa: E731
                                  "parent": parent, "max_model_len": model_cfg.max_model_len}
        return {"object": "list", "data": [card(name, None)] + [card(a, name) for a in adapters]}

    @app.get("/metrics")
    async def metrics():
        if prom is None:
            return error(501, "prometheus_client is not installed", "server_error")
        import prometheus_client as pc
        return PlainTextResponse(pc.generate_latest(prom.registry).decode(), media_type="text/plain; version=0.0.4")

    @app.post("/tokenize")
    async def tokenize(req: Request):
        body = await req.json()
        if tokenizer is None:
            return error(400, "the server runs without a tokenizer")
        ids = list(tokenizer.encode(body.get("prompt", "")))
        return {"tokens": ids, "count": len(ids), "max_model_len": model_cfg.max_model_len}

    @app.post("/detokenize")
    async def detokenize(req: Request):
        body = await req.json()
        if tokenizer is None:
            return error(400, "the server runs without a tokenizer")
        return {"prompt": tokenizer.decode(body.get("tokens", []))}

    async def run_all(prompts: list, sp: SamplingParams, base_id: str, lora=None) -> list[RequestOutput]:
        import asyncio

        async def one(i, p):
            last = None
            async for out in engine.generate(p, sp, f"{base_id}-{i}", lora_request=lora):
                last = out
            finished_metrics(last)
            return last
        return await asyncio.gather(*[one(i, p) for i, p in enumerate(prompts)])

    def normalise_prompts(prompt: Any) -> list:
        if isinstance(prompt, str):
            return [prompt]
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            return [prompt]
        if isinstance(prompt, list) and prompt:
            return list(prompt)
        raise ValueError("prompt must be a string, a list of strings, a list of token ids or a list of those")

    # ---- /v1/completions ----------------------------------------------------------------------
    @app.post("/v1/completions")
    async def completions(req: Request):
        body = await req.json()
        try:
            prompts = normalise_prompts(body.get("prompt"))
            sp = sampling_params_from_request(body)
            lora = pick_adapter(body)
            if tokenizer is None:
                sp.detokenize = False
                if any(isinstance(p, str) for p in prompts):
                    return error(400, "text prompts need a tokenizer; send token ids")
        except (ValueError, TypeError) as e:
            return error(400, str(e))
        rid = "cmpl-" + uuid.uuid4().hex
        created = int(time.time())
        echo = bool(body.get("echo"))

        def choice(out: RequestOutput, p_idx: int, comp, text: str, finish) -> dict:
            plp = out.prompt_logprobs
            if plp is not None:      # JSON object keys are strings
                plp = [None if d is None else {str(t): v for t, v in d.items()} for d in plp]
            return {"index": p_idx * sp.n + comp.index, "text": text, "token_ids": list(comp.token_ids) if tokenizer is None else None,
                    "logprobs": _logprobs_block(comp, tokenizer), "finish_reason": finish, "stop_reason": comp.stop_reason,
                    "prompt_logprobs": plp}

        if body.get("stream"):
            if len(prompts) != 1:
                return error(400, "streaming takes a single prompt")

            async def sse() -> AsyncIterator[str]:
                sent, sent_tokens = {}, {}
                try:
                    async for out in engine.generate(prompts[0], sp, rid + "-0", lora_request=lora):
                        for comp in out.outputs:
                            prev = sent.get(comp.index, 0)
                            delta = comp.text[prev:]
                            sent[comp.index] = len(comp.text)
                            # a chunk per batch of new tokens, also when they add no text yet (an incomplete
                            # multi-byte character, a token outside the tokenizer's table): clients that time the
                            # stream (time to first token, gaps) see every step
                            n_prev = sent_tokens.get(comp.index, 0)
                            new_tokens = len(comp.token_ids) > n_prev
                            sent_tokens[comp.index] = len(comp.token_ids)
                            if delta or new_tokens or comp.finish_reason:
                                chunk = {"id": rid, "object": "text_completion", "created": created, "model": name,
                                         "choices": [{"index": comp.index, "text": delta, "logprobs": None,
                                                      "finish_reason": comp.finish_reason}]}
                                yield f"data: {json.dumps(chunk)}\n\n"
                        if out.finished:
                            finished_metrics(out)
                            yield f"data: {json.dumps({'id': rid, 'object': 'text_completion', 'created': created, 'model': name, 'choices': [], 'usage': _usage(out)})}\n\n"
                except (EngineDeadError, ValueError) as e:
                    yield f"data: {json.dumps({'error': {'message': str(e)}})}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")

        try:
            outs = await run_all(prompts, sp, rid, lora)
        except ValueError as e:
            return error(400, str(e))
        except EngineDeadError as e:
            return error(500, str(e), "server_error")
        choices, usage = [], {"prompt_tokens": 0, "completion_tokens": 0, "total_tokens": 0}
        for i, out in enumerate(outs):
            for comp in out.outputs:
                text = comp.text
                if echo and out.prompt is not None:
                    text = out.prompt + text
                choices.append(choice(out, i, comp, text, comp.finish_reason))
            for k, v in _usage(out).items():
                usage[k] += v
        return {"id": rid, "object": "text_completion", "created": created, "model": name, "choices": choices, "usage": usage}

    # ---- /v1/embeddings, /classify -------------------------------------------------------------
    async def pooled_vectors(body: dict, rid: str):
        """Last-token hidden state of every input (text, token ids, or a list of either)."""
        prompts = normalise_prompts(body.get("input", body.get("prompt")))
        if tokenizer is None and any(isinstance(p, str) for p in prompts):
            raise ValueError("text inputs need a tokenizer; send token ids")
        sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, detokenize=False, pooling=True)
        return await run_all(prompts, sp, rid, pick_adapter(body))

    @app.post("/v1/embeddings")
    async def embeddings(req: Request):
        body = await req.json()
        rid = "embd-" + uuid.uuid4().hex
        try:
            outs = await pooled_vectors(body, rid)
        except (ValueError, TypeError) as e:
            return error(400, str(e))
        except EngineDeadError as e:
            return error(500, str(e), "server_error")
        data, n_tok = [], 0
        for i, out in enumerate(outs):
            vec = out.pooled
            if body.get("normalize", True):
                vec = vec / vec.norm().clamp_min(1e-12)
            data.append({"object": "embedding", "index": i, "embedding": vec.tolist()})
            n_tok += len(out.prompt_token_ids)
        return {"id": rid, "object": "list", "model": name, "data": data,
                "usage": {"prompt_tokens": n_tok, "total_tokens": n_tok}}

    @app.post("/score")
    @app.post("/v1/score")
    async def score(req: Request):
        """Cosine similarity of ``text_1`` with every entry of ``text_2`` (or pairwise for equally long lists)."""
        body = await req.json()
        one = lambda x: isinstance(x, str) or (isinstance(x, list) and x and isinstance(x[0], int))   # noqa: E731
        a = [body.get("text_1")] if one(body.get("text_1")) else list(body.get("text_1") or [])
        b = [body.get("text_2")] if one(body.get("text_2")) else list(body.get("text_2") or [])
        if len(a) == 1 and len(b) > 1:
            a = a * len(b)
        if not a or len(a) != len(b):
            return error(400, "score takes one-to-many or equally long lists in text_1 / text_2")
        rid = "score-" + uuid.uuid4().hex
        try:
            outs = await pooled_vectors({**body, "input": a + b}, rid)
        except (ValueError, TypeError) as e:
            return error(400, str(e))
        except EngineDeadError as e:
            return error(500, str(e), "server_error")
        vecs = [o.pooled / o.pooled.norm().clamp_min(1e-12) for o in outs]
        data = [{"index": i, "object": "score", "score": float((vecs[i] * vecs[len(a) + i]).sum())} for i in range(len(a))]
        return {"id": rid, "object": "list", "model": name, "data": data}

    score_head = {}

    @app.post("/classify")
    async def classify(req: Request):
        body = await req.json()
        import torch
        if "w" not in score_head:
            from ..models.loader import iter_checkpoint
            path = engine.engine.config.model.path
            for tname, tensor in (iter_checkpoint(path) if path else ()):
                if tname in ("score.weight", "classifier.weight"):
                    score_head["w"] = tensor.float()
                    break
        if "w" not in score_head:
            return error(400, "the served checkpoint has no sequence-classification head (score.weight)")
        rid = "cls-" + uuid.uuid4().hex
        try:
            outs = await pooled_vectors(body, rid)
        except (ValueError, TypeError) as e:
            return error(400, str(e))
        except EngineDeadError as e:
            return error(500, str(e), "server_error")
        data = []
        for i, out in enumerate(outs):
            probs = torch.softmax(out.pooled.float() @ score_head["w"].t(), dim=-1)
            data.append({"index": i, "label": int(probs.argmax()), "probs": probs.tolist()})
        return {"id": rid, "object": "list", "model": name, "data": data}

    # ---- /v1/chat/completions -----------------------------------------------------------------
    def chat_prompt(messages: list, add_generation_prompt: bool = True, tools: Optional[list] = None) -> str:
        if hasattr(tokenizer, "apply_chat_template") and getattr(tokenizer, "chat_template", None):
            kw = {"tools": tools} if tools else {}
            return tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt,
                                                 **kw)
        text = ""
        if tools:
            from .tool_calls import describe_tools
            text = "system: " + describe_tools(tools) + "\n"
        for m in messages:
            content = m.get("content")
            if content is None and m.get("tool_calls"):
                content = json.dumps([c.get("function", c) for c in m["tool_calls"]])
            text += f"{m['role']}: {content}\n"
        return text + ("assistant: " if add_generation_prompt else "")

    @app.post("/v1/chat/completions")
    async def chat(req: Request):
        body = await req.json()
        if tokenizer is None:
            return error(400, "chat completions need a tokenizer")
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs:
            return error(400, "messages must be a non-empty list")
        tools = body.get("tools") if body.get("tool_choice") != "none" else None
        tool_choice = body.get("tool_choice", "auto" if tools else None)
        try:
            from . import tool_calls as tc
            sp = sampling_params_from_request(body, default_max_tokens=256)
            forced = tc.forced_schema(tools, tool_choice) if tools else None
            if forced is not None:
                sp.guided_json, sp.guided_regex = forced, None      # the call's arguments always parse
            prompt = chat_prompt(msgs, body.get("add_generation_prompt", True), tools)
            lora = pick_adapter(body)
        except (ValueError, TypeError, KeyError) as e:
            return error(400, str(e))
        rid = "chatcmpl-" + uuid.uuid4().hex
        created = int(time.time())

        def message_of(comp) -> tuple[dict, Optional[str]]:
            """Assistant message (with tool calls where the text holds some) and the finish reason."""
            text, reasoning = comp.text, None
            if reasoning_parser and forced is None:
                reasoning, text = tc.split_reasoning(text)
            if not tools:
                msg = {"role": "assistant", "content": text}
                if reasoning:
                    msg["reasoning_content"] = reasoning
                return msg, comp.finish_reason
            if forced is not None:
                try:
                    calls, content = tc.calls_from_forced(comp.text, tools, tool_choice), None
                except (ValueError, KeyError, TypeError):      # cut off by max_tokens before the JSON closed
                    calls, content = [], comp.text
            else:
                content, calls = tc.calls_from_text(text or "", tools, tool_call_parser)
            msg = {"role": "assistant", "content": content}
            if reasoning:
                msg["reasoning_content"] = reasoning
            if calls:
                msg["tool_calls"] = calls
            return msg, ("tool_calls" if calls and comp.finish_reason == "stop" else comp.finish_reason)

        if body.get("stream") and tools:
            # calls are recognised on the complete text: one chunk with the whole message, then the end marker
            async def sse_tools() -> AsyncIterator[str]:
                try:
                    out = (await run_all([prompt], sp, rid, lora))[0]
                    for c in out.outputs:
                        msg, fin = message_of(c)
                        chunk = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": name,
                                 "choices": [{"index": c.index, "delta": msg, "finish_reason": fin}]}
                        yield f"data: {json.dumps(chunk)}\n\n"
                except (EngineDeadError, ValueError) as e:
                    yield f"data: {json.dumps({'error': {'message': str(e)}})}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse_tools(), media_type="text/event-stream")
        if body.get("stream"):
            async def sse() -> AsyncIterator[str]:
                sent = {}
                first = True
                try:
                    async for out in engine.generate(prompt, sp, rid, lora_request=lora):
                        for comp in out.outputs:
                            prev = sent.get(comp.index, 0)
                            delta = comp.text[prev:]
                            sent[comp.index] = len(comp.text)
                            d = {"content": delta}
                            if first:
                                d["role"] = "assistant"
                                first = False
                            if delta or comp.finish_reason:
                                chunk = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": name,
                                         "choices": [{"index": comp.index, "delta": d, "finish_reason": comp.finish_reason}]}
                                yield f"data: {json.dumps(chunk)}\n\n"
                        if out.finished:
                            finished_metrics(out)
                except (EngineDeadError, ValueError) as e:
                    yield f"data: {json.dumps({'error': {'message': str(e)}})}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        try:
            out = (await run_all([prompt], sp, rid, lora))[0]
        except ValueError as e:
            return error(400, str(e))
        except EngineDeadError as e:
            return error(500, str(e), "server_error")
        choices = []
        for c in out.outputs:
            msg, fin = message_of(c)
            choices.append({"index": c.index, "message": msg, "logprobs": _logprobs_block(c, tokenizer),
                            "finish_reason": fin})
        return {"id": rid, "object": "chat.completion", "created": created, "model": name, "choices": choices,
                "usage": _usage(out)}

    return app


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--chat-template", default=None, help="a Jinja chat template (file or literal) replacing the tokenizer's")
    ap.add_argument("--tool-call-parser", default="auto",
                    help="spelling of tool calls in free text: auto, hermes, llama3_json, mistral, pythonic")
    ap.add_argument("--enable-auto-tool-choice", action="store_true",
                    help="accepted for command lines written for the reference's server (tool_choice=auto is always on)")
    ap.add_argument("--reasoning-parser", default=None, choices=["deepseek_r1"],
                    help="move <think> ... </think> blocks of chat answers into reasoning_content")
    ap.add_argument("--api-key", default=os.environ.get("TW_API_KEY"),
                    help="require 'Authorization: Bearer <key>' on the /v1 routes (default: the TW_API_KEY variable)")
    ap.add_argument("--allowed-origins", nargs="*", default=None, help="origins to answer with CORS headers")
    ap.add_argument("--lora-modules", nargs="*", default=[], metavar="NAME=PATH",
                    help="adapters to serve; a request selects one by its name in the model field (needs --enable-lora)")
    EngineArgs.add_cli_args(ap)
    ns = ap.parse_args()
    args = EngineArgs.from_cli_args(ns)
    lora_modules = dict(m.split("=", 1) for m in ns.lora_modules)
    if lora_modules:
        args.enable_lora = True
    if args.tensor_parallel_size > 1 and args.distributed_executor_backend == "auto":
        args.distributed_executor_backend = "mp"
    if args.data_parallel_size > 1:
        from ..engine.data_parallel import DataParallelEngine
        engine = DataParallelEngine.from_engine_args(args)
    else:
        engine = AsyncLLMEngine.from_engine_args(args)
    if ns.chat_template and engine.engine.tokenizer is not None:
        import os as _os
        tpl = open(ns.chat_template).read() if _os.path.exists(ns.chat_template) else ns.chat_template
        engine.engine.tokenizer.chat_template = tpl
    import uvicorn
    try:
        uvicorn.run(build_app(engine, ns.served_model_name, lora_modules, ns.tool_call_parser, ns.reasoning_parser,
                              ns.api_key, ns.allowed_origins),
                    host=ns.host, port=ns.port, log_level="info")
    finally:
        engine.shutdown()


if __name__ == "__main__":
    main()
