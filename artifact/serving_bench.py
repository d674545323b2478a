#!/usr/bin/env python
"""Online serving benchmark against the OpenAI-compatible server (the counterpart of the reference's
``benchmarks/benchmark_serving.py``): requests with random token-id prompts arrive as a Poisson process of
``--request-rate`` per second (``inf``: all at once), each is streamed from ``/v1/completions``, and the client
reports request / token throughput and the mean, median and 99th percentile of the time to the first token (TTFT),
the time per output token after the first (TPOT), the gaps between streamed chunks (ITL) and the end-to-end
latency. ``--max-concurrency`` bounds the requests in flight.

    python -m tokenweave_b200.entrypoints.api_server --model llama-3.1-8b --port 8000 &
    python artifact/serving_bench.py --base-url http://127.0.0.1:8000 --num-prompts 200 --request-rate 8

``--spawn-server "<server arguments>"`` starts the server itself (on ``--port``), waits for ``/health`` and stops it
afterwards."""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import random
import subprocess
import sys
import time
from dataclasses import dataclass, field
from typing import Optional

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import RESULTS_DIR, write_rows  # noqa: E402


@dataclass
class RequestRecord:
    ok: bool = False
    error: str = ""
    prompt_tokens: int = 0
    output_tokens: int = 0
    start: float = 0.0
    ttft: float = 0.0
    latency: float = 0.0
    gaps: list[float] = field(default_factory=list)


def percentile(values: list[float], q: float) -> float:
    if not values:
        return float("nan")
    xs = sorted(values)
    k = (len(xs) - 1) * q
    lo, hi = int(k), min(int(k) + 1, len(xs) - 1)
    return xs[lo] + (xs[hi] - xs[lo]) * (k - lo)


def summarise(records: list[RequestRecord], elapsed: float) -> dict:
    """Throughput and latency statistics of the completed requests (seconds -> milliseconds for the latencies)."""
    good = [r for r in records if r.ok]
    ttft = [r.ttft * 1e3 for r in good]
    tpot = [(r.latency - r.ttft) / (r.output_tokens - 1) * 1e3 for r in good if r.output_tokens > 1]
    itl = [g * 1e3 for r in good for g in r.gaps]
    e2e = [r.latency * 1e3 for r in good]
    out = {"completed": len(good), "failed": len(records) - len(good), "elapsed_s": elapsed,
           "requests_per_s": len(good) / elapsed if elapsed > 0 else 0.0,
           "output_tokens_per_s": sum(r.output_tokens for r in good) / elapsed if elapsed > 0 else 0.0,
           "total_tokens_per_s": sum(r.output_tokens + r.prompt_tokens for r in good) / elapsed if elapsed > 0 else 0.0}
    for name, xs in (("ttft", ttft), ("tpot", tpot), ("itl", itl), ("e2e", e2e)):
        out[f"{name}_mean_ms"] = sum(xs) / len(xs) if xs else float("nan")
        out[f"{name}_median_ms"] = percentile(xs, 0.5)
        out[f"{name}_p99_ms"] = percentile(xs, 0.99)
    return out


async def one_request(session, url: str, body: dict, rec: RequestRecord) -> None:
    """Streams one completion and fills ``rec``; the server's last chunk carries the token counts."""
    rec.start = time.perf_counter()
    last = rec.start
    try:
        async with session.post(url, json=body) as resp:
            if resp.status != 200:
                rec.error = f"HTTP {resp.status}: {(await resp.text())[:200]}"
                return
            buf = b""
            async for piece in resp.content.iter_any():
                buf += piece
                while b"\n\n" in buf:
                    event, buf = buf.split(b"\n\n", 1)
                    if not event.startswith(b"data: "):
                        continue
                    payload = event[6:]
                    if payload == b"[DONE]":
                        continue
                    msg = json.loads(payload)
                    if "error" in msg:
                        rec.error = str(msg["error"])
                        return
                    now = time.perf_counter()
                    if msg.get("choices"):
                        if rec.ttft == 0.0:
                            rec.ttft = now - rec.start
                        else:
                            rec.gaps.append(now - last)
                        last = now
                    if "usage" in msg:
                        rec.prompt_tokens = msg["usage"]["prompt_tokens"]
                        rec.output_tokens = msg["usage"]["completion_tokens"]
            rec.latency = time.perf_counter() - rec.start
            if rec.ttft == 0.0:              # nothing but the final chunk came back (no text deltas)
                rec.ttft = rec.latency
            rec.ok = rec.output_tokens > 0
            if not rec.ok and not rec.error:
                rec.error = "no usage block in the stream"
    except Exception as e:  # connection errors end the request, not the run
        rec.error = f"{type(e).__name__}: {e}"


async def run(base_url: str, model: Optional[str], num_prompts: int, request_rate: float, input_len: int,
              output_len: int, vocab: int, max_concurrency: int = 0, seed: int = 0, temperature: float = 0.0) -> dict:
    """Fires the requests and returns ``summarise``'s dictionary."""
    import aiohttp
    rng = random.Random(seed)
    prompts = [[rng.randrange(1, vocab) for _ in range(input_len)] for _ in range(num_prompts)]
    sem = asyncio.Semaphore(max_concurrency) if max_concurrency > 0 else None
    records = [RequestRecord() for _ in prompts]
    url = base_url.rstrip("/") + "/v1/completions"

    async def guarded(session, body, rec):
        if sem is None:
            await one_request(session, url, body, rec)
        else:
            async with sem:
                await one_request(session, url, body, rec)

    timeout = aiohttp.ClientTimeout(total=None, sock_read=600)
    async with aiohttp.ClientSession(timeout=timeout) as session:
        t0 = time.perf_counter()
        tasks = []
        for prompt, rec in zip(prompts, records):
            body = {"prompt": prompt, "max_tokens": output_len, "temperature": temperature, "ignore_eos": True,
                    "stream": True}
            if model:
                body["model"] = model
            tasks.append(asyncio.create_task(guarded(session, body, rec)))
            if request_rate != float("inf"):
                await asyncio.sleep(rng.expovariate(request_rate))        # Poisson arrivals
        await asyncio.gather(*tasks)
        elapsed = time.perf_counter() - t0
    res = summarise(records, elapsed)
    res["first_error"] = next((r.error for r in records if r.error), "")
    return res


def wait_for_health(base_url: str, seconds: float) -> bool:
    import urllib.request
    deadline = time.time() + seconds
    while time.time() < deadline:
        try:
            with urllib.request.urlopen(base_url.rstrip("/") + "/health", timeout=2) as r:
                if r.status == 200:
                    return True
        except Exception:
            time.sleep(0.5)
    return False


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default=None, help="default: http://127.0.0.1:<--port>")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--model", default=None, help="served model name to put into the requests")
    ap.add_argument("--num-prompts", type=int, default=200)
    ap.add_argument("--request-rate", type=float, default=float("inf"), help="requests per second (inf: all at once)")
    ap.add_argument("--input-len", type=int, default=512)
    ap.add_argument("--output-len", type=int, default=128)
    ap.add_argument("--vocab-size", type=int, default=32000, help="token ids of the random prompts are below this")
    ap.add_argument("--max-concurrency", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--spawn-server", default=None, help="arguments for tokenweave_b200.entrypoints.api_server")
    ap.add_argument("--server-start-timeout", type=float, default=600.0)
    ap.add_argument("--out", default=os.path.join(RESULTS_DIR, "serving_bench"))
    args = ap.parse_args()
    base = args.base_url or f"http://127.0.0.1:{args.port}"
    server = None
    if args.spawn_server is not None:
        cmd = [sys.executable, "-m", "tokenweave_b200.entrypoints.api_server", "--host", "127.0.0.1", "--port",
               str(args.port)] + args.spawn_server.split()
        server = subprocess.Popen(cmd)
    try:
        if not wait_for_health(base, args.server_start_timeout if server else 10.0):
            raise SystemExit(f"no server answering at {base}/health")
        res = asyncio.run(run(base, args.model, args.num_prompts, args.request_rate, args.input_len, args.output_len,
                              args.vocab_size, args.max_concurrency, args.seed, args.temperature))
    finally:
        if server is not None:
            server.terminate()
            try:
                server.wait(timeout=30)
            except subprocess.TimeoutExpired:
                server.kill()
    row = {"num_prompts": args.num_prompts, "request_rate": args.request_rate, "input_len": args.input_len,
           "output_len": args.output_len, "max_concurrency": args.max_concurrency, **res}
    print("============ Serving Benchmark Result ============")
    for k, v in row.items():
        print(f"{k:<24}{v:.2f}" if isinstance(v, float) else f"{k:<24}{v}")
    write_rows(args.out, "serving_bench", [row])


if __name__ == "__main__":
    main()
