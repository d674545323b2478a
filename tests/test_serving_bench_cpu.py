"""The online serving benchmark client against a live server (tiny random-weight model on CPU, uvicorn on a
thread): every request streams back, token counts come from the final chunk, latency statistics are filled in."""
import asyncio
import os
import sys
import threading
import time

import pytest

pytest.importorskip("fastapi")
pytest.importorskip("aiohttp")
uvicorn = pytest.importorskip("uvicorn")

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "artifact"))

from tw_testing import free_port  # noqa: E402


def test_serving_benchmark_against_a_live_server():
    import serving_bench
    from tokenweave_b200.config import EngineArgs
    from tokenweave_b200.engine.async_engine import AsyncLLMEngine
    from tokenweave_b200.entrypoints.api_server import build_app
    engine = AsyncLLMEngine.from_engine_args(EngineArgs(model="tiny-llama", dtype="float32", device="cpu", block_size=16,
                                                        max_num_batched_tokens=128, seed=1))
    port = free_port()
    server = uvicorn.Server(uvicorn.Config(build_app(engine, "tiny"), host="127.0.0.1", port=port, log_level="error"))
    thread = threading.Thread(target=server.run, daemon=True)
    thread.start()
    try:
        base = f"http://127.0.0.1:{port}"
        assert serving_bench.wait_for_health(base, 30.0)
        # token ids above the byte tokenizer's 256 byte values: they add no text, and the stream must still carry a
        # chunk per step for the client to time
        res = asyncio.run(serving_bench.run(base, "tiny", num_prompts=6, request_rate=50.0, input_len=20, output_len=8,
                                            vocab=1000, max_concurrency=4, seed=3))
        assert res["completed"] == 6 and res["failed"] == 0, res
        assert res["output_tokens_per_s"] > 0 and res["total_tokens_per_s"] > res["output_tokens_per_s"]
        for key in ("ttft_mean_ms", "e2e_median_ms", "e2e_p99_ms", "tpot_mean_ms"):
            assert res[key] == res[key] and res[key] > 0, (key, res)          # not NaN
        assert res["ttft_median_ms"] < res["e2e_median_ms"]
        assert res["itl_mean_ms"] == res["itl_mean_ms"] and res["itl_mean_ms"] > 0      # gaps between chunks were seen
        # a request the server refuses is counted, not fatal
        bad = asyncio.run(serving_bench.run(base, "tiny", num_prompts=2, request_rate=float("inf"), input_len=5000,
                                            output_len=4, vocab=250))
        assert bad["completed"] == 0 and bad["failed"] == 2 and bad["first_error"]
    finally:
        server.should_exit = True
        thread.join(timeout=20)
        engine.shutdown()


def test_percentiles_and_summary():
    import serving_bench
    assert serving_bench.percentile([1.0, 2.0, 3.0, 4.0], 0.5) == 2.5
    assert serving_bench.percentile([5.0], 0.99) == 5.0
    recs = [serving_bench.RequestRecord(ok=True, prompt_tokens=10, output_tokens=5, ttft=0.1, latency=0.5, gaps=[0.1] * 4),
            serving_bench.RequestRecord(ok=False, error="x")]
    s = serving_bench.summarise(recs, 2.0)
    assert s["completed"] == 1 and s["failed"] == 1 and s["output_tokens_per_s"] == 2.5
    assert abs(s["tpot_mean_ms"] - 100.0) < 1e-6 and abs(s["itl_p99_ms"] - 100.0) < 1e-6
