"""Data-parallel serving on CPU: two engine replicas behind one front end give the outputs of a single engine,
share the load, and sit behind the HTTP server like one engine."""
import asyncio

import pytest

from tokenweave_b200 import LLM, SamplingParams
from tokenweave_b200.config import EngineArgs
from tokenweave_b200.engine.data_parallel import DataParallelEngine

ARGS = dict(model="tiny-llama", dtype="float32", device="cpu", block_size=16, max_num_batched_tokens=128, seed=1,
            skip_tokenizer_init=True)


def test_two_replicas_match_one_engine_and_share_the_load():
    prompts = [[(7 * i + j) % 1000 for j in range(5 + i)] for i in range(8)]
    sp = SamplingParams(temperature=0, max_tokens=6, ignore_eos=True)
    single = LLM(**ARGS)
    want = [o.outputs[0].token_ids for o in single.generate(prompts, sp)]
    single.shutdown()
    dp = DataParallelEngine.from_engine_args(EngineArgs(data_parallel_size=2, **ARGS))
    assert [r.engine.config.parallel.data_parallel_rank for r in dp.replicas] == [0, 1]
    assert dp.replicas[1].engine.config.parallel.device_offset == 1

    async def run():
        async def one(i, p):
            last = None
            async for out in dp.generate(p, sp, f"r{i}"):
                last = out
            return last.outputs[0].token_ids
        got = await asyncio.gather(*[one(i, p) for i, p in enumerate(prompts)])
        # an aborted stream frees its slot in the balancer
        agen = dp.generate(prompts[0], SamplingParams(temperature=0, max_tokens=500, ignore_eos=True), "gone")
        async for _ in agen:
            break
        await agen.aclose()
        return got

    try:
        got = asyncio.run(run())
        assert got == want
        assert sum(dp.served) == 9 and min(dp.served) >= 3, dp.served
        assert dp.in_flight == [0, 0]
        assert dp.is_running
    finally:
        dp.shutdown()


def test_server_on_top_of_replicas():
    pytest.importorskip("fastapi")
    pytest.importorskip("httpx")
    from starlette.testclient import TestClient
    from tokenweave_b200.entrypoints.api_server import build_app
    args = dict(ARGS, skip_tokenizer_init=False)
    dp = DataParallelEngine.from_engine_args(EngineArgs(data_parallel_size=2, **args))
    try:
        with TestClient(build_app(dp, "tiny")) as c:
            body = {"prompt": ["hello", "world", "again"], "max_tokens": 4, "temperature": 0, "ignore_eos": True}
            r = c.post("/v1/completions", json=body)
            assert r.status_code == 200, r.text
            assert len(r.json()["choices"]) == 3 and r.json()["usage"]["completion_tokens"] == 12
            assert c.get("/health").json() == {"status": "ok"}
        assert min(dp.served) >= 1
    finally:
        dp.shutdown()
