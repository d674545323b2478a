"""OpenAI-compatible server and the asynchronous engine front on CPU (tiny random-weight model, byte
tokenizer): completions, chat, streaming, token-id prompts, aborts, metrics."""
import asyncio
import json

import pytest

from tokenweave_b200 import SamplingParams
from tokenweave_b200.config import EngineArgs
from tokenweave_b200.engine.async_engine import AsyncLLMEngine

fastapi = pytest.importorskip("fastapi")
pytest.importorskip("httpx")


@pytest.fixture(scope="module")
def engine():
    eng = AsyncLLMEngine.from_engine_args(EngineArgs(model="tiny-llama", dtype="float32", device="cpu", block_size=16,
                                                     max_num_batched_tokens=128, seed=1))
    yield eng
    eng.shutdown()


@pytest.fixture(scope="module")
def client(engine):
    from starlette.testclient import TestClient
    from tokenweave_b200.entrypoints.api_server import build_app
    with TestClient(build_app(engine, "tiny")) as c:
        yield c


def test_health_models_tokenize(client):
    assert client.get("/health").json() == {"status": "ok"}
    models = client.get("/v1/models").json()
    assert models["data"][0]["id"] == "tiny"
    tok = client.post("/tokenize", json={"prompt": "hi"}).json()
    assert tok["tokens"] == [256, 104, 105] and tok["count"] == 3
    assert client.post("/detokenize", json={"tokens": [104, 105]}).json()["prompt"] == "hi"


def test_completion_matches_offline_engine(client, engine):
    body = {"model": "tiny", "prompt": "hello world", "max_tokens": 6, "temperature": 0, "ignore_eos": True, "logprobs": 2}
    r = client.post("/v1/completions", json=body)
    assert r.status_code == 200, r.text
    data = r.json()
    assert data["object"] == "text_completion" and len(data["choices"]) == 1
    ch = data["choices"][0]
    assert ch["finish_reason"] == "length"
    assert data["usage"] == {"prompt_tokens": 12, "completion_tokens": 6, "total_tokens": 18}
    assert len(ch["logprobs"]["token_logprobs"]) == 6 and all(len(t) >= 1 for t in ch["logprobs"]["top_logprobs"])
    # the same request again is deterministic, and a batch of prompts keeps its order
    again = client.post("/v1/completions", json=body).json()["choices"][0]["text"]
    assert again == ch["text"]
    both = client.post("/v1/completions", json={**body, "prompt": ["hello world", "abc"], "logprobs": None}).json()
    assert [c["index"] for c in both["choices"]] == [0, 1] and both["choices"][0]["text"] == ch["text"]
    # token-id prompt
    ids = client.post("/v1/completions", json={"prompt": [256, 104, 105], "max_tokens": 3, "temperature": 0}).json()
    assert ids["usage"]["prompt_tokens"] == 3 and ids["choices"][0]["prompt_logprobs"] is None
    plp = client.post("/v1/completions", json={"prompt": [256, 104, 105], "max_tokens": 1, "temperature": 0,
                                               "prompt_logprobs": 2}).json()["choices"][0]["prompt_logprobs"]
    assert plp[0] is None and "104" in plp[1] and "105" in plp[2] and all(v <= 0 for v in plp[1].values())


def test_streaming_completion_concatenates_to_the_full_text(client):
    body = {"prompt": "stream me", "max_tokens": 8, "temperature": 0, "ignore_eos": True}
    full = client.post("/v1/completions", json=body).json()["choices"][0]["text"]
    text, done, usage = "", False, None
    with client.stream("POST", "/v1/completions", json={**body, "stream": True}) as r:
        assert r.status_code == 200
        for line in r.iter_lines():
            if not line.startswith("data: "):
                continue
            payload = line[len("data: "):]
            if payload == "[DONE]":
                done = True
                break
            chunk = json.loads(payload)
            for c in chunk["choices"]:
                text += c["text"]
            usage = chunk.get("usage", usage)
    assert done and text == full and usage["completion_tokens"] == 8


def test_chat_completion_and_stream(client):
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    r = client.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 5, "temperature": 0, "ignore_eos": True})
    assert r.status_code == 200, r.text
    data = r.json()
    assert data["object"] == "chat.completion" and data["choices"][0]["message"]["role"] == "assistant"
    assert data["usage"]["completion_tokens"] == 5
    pieces = []
    with client.stream("POST", "/v1/chat/completions", json={"messages": msgs, "max_tokens": 5, "temperature": 0,
                                                             "ignore_eos": True, "stream": True}) as s:
        for line in s.iter_lines():
            if line.startswith("data: ") and line != "data: [DONE]":
                pieces.append(json.loads(line[6:])["choices"][0]["delta"].get("content", ""))
    assert "".join(pieces) == data["choices"][0]["message"]["content"]


def test_bad_requests_are_rejected_and_the_server_keeps_serving(client):
    assert client.post("/v1/completions", json={"prompt": "x", "temperature": -1}).status_code == 400
    assert client.post("/v1/completions", json={"prompt": [999999], "max_tokens": 2}).status_code == 400
    assert client.post("/v1/chat/completions", json={"messages": []}).status_code == 400
    assert client.post("/v1/completions", json={"prompt": "still alive", "max_tokens": 2}).status_code == 200
    m = client.get("/metrics")
    assert m.status_code == 200 and "tokenweave:generation_tokens_total" in m.text


def test_embeddings_endpoint_matches_the_offline_api(client):
    import torch
    from tokenweave_b200 import LLM
    r = client.post("/v1/embeddings", json={"input": ["hello world", "abc"]})
    assert r.status_code == 200, r.text
    data = r.json()["data"]
    assert [d["index"] for d in data] == [0, 1] and r.json()["usage"]["prompt_tokens"] == 12 + 4
    llm = LLM("tiny-llama", dtype="float32", device="cpu", block_size=16, max_num_batched_tokens=128, seed=1)
    want = llm.embed(["hello world", "abc"])
    llm.shutdown()
    for d, w in zip(data, want):
        assert torch.allclose(torch.tensor(d["embedding"]), w.data, atol=1e-5)
    raw = client.post("/v1/embeddings", json={"input": [256, 104, 105], "normalize": False}).json()["data"][0]["embedding"]
    assert abs(sum(x * x for x in raw) ** 0.5 - 1.0) > 1e-3          # not normalised
    assert client.post("/classify", json={"input": "x"}).status_code == 400     # no classification head here


def test_adapter_selected_by_model_name(tmp_path):
    from starlette.testclient import TestClient
    from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
    from tokenweave_b200.entrypoints.api_server import build_app
    from test_lora_cpu import _make_adapter
    from tw_testing import make_hf_state
    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    _make_adapter(str(tmp_path / "ad"), cfg, make_hf_state(cfg, seed=0), r=4, alpha=64, seed=3)
    eng = AsyncLLMEngine.from_engine_args(EngineArgs(model="tiny-llama", dtype="float32", device="cpu", block_size=16,
                                                     max_num_batched_tokens=128, seed=1, enable_lora=True))
    try:
        with TestClient(build_app(eng, "tiny", {"tiny-ad": str(tmp_path / "ad")})) as c:
            assert [m["id"] for m in c.get("/v1/models").json()["data"]] == ["tiny", "tiny-ad"]
            body = {"prompt": "hello world", "max_tokens": 8, "temperature": 0, "ignore_eos": True, "logprobs": 1}
            base = c.post("/v1/completions", json={**body, "model": "tiny"}).json()["choices"][0]
            ad = c.post("/v1/completions", json={**body, "model": "tiny-ad"}).json()["choices"][0]
            assert ad["logprobs"]["token_logprobs"] != base["logprobs"]["token_logprobs"]
            again = c.post("/v1/completions", json={**body, "model": "tiny"}).json()["choices"][0]
            assert again["logprobs"]["token_logprobs"] == base["logprobs"]["token_logprobs"]
            assert c.post("/v1/completions", json={**body, "model": "nobody"}).status_code == 400
    finally:
        eng.shutdown()


def test_async_engine_abort_frees_the_request(engine):
    async def run():
        agen = engine.generate([1, 2, 3, 4], SamplingParams(temperature=0, max_tokens=10_000, ignore_eos=True), "abort-me")
        n = 0
        async for out in agen:
            n += 1
            if n == 3:
                break
        await agen.aclose()                 # the consumer walks away: the request must be aborted
        for _ in range(200):
            if not engine.engine.has_unfinished_requests():
                return True
            await asyncio.sleep(0.01)
        return False
    assert asyncio.run(run())


def test_score_version_and_stop_string_options(client):
    assert client.get("/ping").json() == {"status": "ok"} and "version" in client.get("/version").json()
    r = client.post("/v1/score", json={"text_1": "hello", "text_2": ["hello", "something else"]})
    assert r.status_code == 200, r.text
    scores = [d["score"] for d in r.json()["data"]]
    assert abs(scores[0] - 1.0) < 1e-5 and scores[1] < 0.9999
    assert client.post("/score", json={"text_1": ["a", "b"], "text_2": ["c"]}).status_code == 400
    # stop strings: cut before the match by default, kept with include_stop_str_in_output
    body = {"prompt": "stop test", "max_tokens": 12, "temperature": 0, "ignore_eos": True}
    full = client.post("/v1/completions", json=body).json()["choices"][0]["text"]
    needle = full[4:6]
    cut = client.post("/v1/completions", json={**body, "stop": [needle]}).json()["choices"][0]
    kept = client.post("/v1/completions", json={**body, "stop": [needle], "include_stop_str_in_output": True}).json()["choices"][0]
    assert cut["finish_reason"] == "stop" and full.startswith(cut["text"]) and needle not in cut["text"]
    assert kept["text"] == cut["text"] + needle


def test_api_key_and_cors(engine):
    from starlette.testclient import TestClient
    from tokenweave_b200.entrypoints.api_server import build_app
    with TestClient(build_app(engine, "tiny", api_key="s3cret", allowed_origins=["https://ui.example"])) as c:
        body = {"prompt": "hi", "max_tokens": 2, "temperature": 0}
        assert c.get("/health").status_code == 200                        # liveness needs no key
        assert c.post("/v1/completions", json=body).status_code == 401
        assert c.post("/v1/completions", json=body, headers={"Authorization": "Bearer wrong"}).status_code == 401
        ok = c.post("/v1/completions", json=body, headers={"Authorization": "Bearer s3cret"})
        assert ok.status_code == 200 and ok.json()["choices"][0]["finish_reason"] == "length"
        assert c.get("/v1/models", headers={"Authorization": "Bearer s3cret"}).status_code == 200
        pre = c.options("/v1/completions", headers={"Origin": "https://ui.example",
                                                    "Access-Control-Request-Method": "POST"})
        assert pre.headers.get("access-control-allow-origin") == "https://ui.example"
