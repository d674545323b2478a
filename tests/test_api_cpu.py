"""Offline API extras on CPU: chat, sleep / wake-up, sharded state, request tracing, metrics, CLI flags."""
import argparse
import json

import pytest
import torch

from tokenweave_b200 import LLM, SamplingParams
from tokenweave_b200.config import EngineArgs


def _llm(**kw):
    args = dict(dtype="float32", device="cpu", tokenizer="byte", block_size=16, max_num_batched_tokens=256)
    args.update(kw)
    return LLM("tiny-llama", **args)


def test_chat_uses_transcript_template():
    llm = _llm()
    out = llm.chat([{"role": "user", "content": "hi"}], SamplingParams(temperature=0, max_tokens=4))[0]
    assert out.prompt == "user: hi\nassistant: " and len(out.outputs[0].token_ids) == 4


def test_sleep_wake_up_and_sharded_state(tmp_path):
    llm = _llm()
    sp = SamplingParams(temperature=0, max_tokens=6)
    before = llm.generate("abc", sp)[0].outputs[0].token_ids
    worker = llm.llm_engine.core.executor.worker
    llm.sleep(level=1)
    assert all(p.numel() == 0 for p in worker.runner.model.parameters())
    assert worker.runner.model.layers[0].attn.k_cache is None
    llm.wake_up()
    assert llm.generate("abc", sp)[0].outputs[0].token_ids == before
    llm.save_sharded_state(str(tmp_path))
    for p in worker.runner.model.parameters():
        p.data.zero_()
    worker.load_sharded_state(str(tmp_path))
    assert llm.generate("abc", sp)[0].outputs[0].token_ids == before


def test_request_tracer_jsonl(tmp_path):
    from tokenweave_b200.utils.tracing import SPAN_ATTRS, RequestTracer
    llm = _llm()
    out = llm.generate("hello", SamplingParams(temperature=0, max_tokens=3))[0]
    path = tmp_path / "spans.jsonl"
    tracer = RequestTracer(jsonl_path=str(path))
    tracer.record(out)
    tracer.close()
    span = json.loads(path.read_text().splitlines()[0])
    assert set(span["attributes"]) == set(SPAN_ATTRS)
    assert span["attributes"]["gen_ai.usage.completion_tokens"] == 3
    assert span["attributes"]["gen_ai.latency.e2e"] >= span["attributes"]["gen_ai.latency.time_to_first_token"] >= 0


def test_stat_loggers():
    from tokenweave_b200.utils.metrics import LoggingStatLogger, PrometheusStatLogger, StepStats
    lg = LoggingStatLogger(interval_s=0.0)
    lg.record(StepStats(num_tokens=100, num_running=2, num_waiting=1, kv_usage=0.5, num_generated=2))
    pm = PrometheusStatLogger("tiny")
    pm.record(StepStats(num_tokens=64, num_running=1, num_waiting=0, kv_usage=0.25, num_generated=1))
    pm.record_finished(0.1, 0.5)
    import prometheus_client
    text = prometheus_client.generate_latest(pm.registry).decode()
    assert "tokenweave:prompt_tokens_total" in text and "tokenweave:kv_cache_usage" in text


def test_engine_args_cli_round_trip():
    parser = EngineArgs.add_cli_args(argparse.ArgumentParser())
    ns = parser.parse_args(["--model", "tiny-qwen2", "--tensor-parallel-size", "2", "--max-num-batched-tokens", "4096",
                            "--tokenweave-mode", "fuse_only", "--no-enable-chunked-prefill"])
    args = EngineArgs.from_cli_args(ns)
    cfg = args.create_engine_config()
    assert cfg.model.architecture == "qwen2" and cfg.model.qkv_bias
    assert cfg.parallel.tensor_parallel_size == 2 and cfg.scheduler.max_num_batched_tokens == 4096
    assert cfg.tokenweave.mode == "fuse_only" and cfg.scheduler.enable_chunked_prefill is False


def test_beam_search_finds_the_most_likely_continuation():
    """Width-1 beam search is greedy decoding; a wider beam never scores below it, and the returned
    cumulative log-probabilities equal the sum of the model's per-step log-probabilities."""
    from tokenweave_b200 import BeamSearchParams, LLM, SamplingParams
    llm = LLM("tiny-llama", dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16,
              max_num_batched_tokens=256, enable_prefix_caching=True, seed=5)
    prompt = list(range(3, 20))
    greedy = llm.generate([prompt], SamplingParams(temperature=0, max_tokens=5, ignore_eos=True, logprobs=1))[0].outputs[0]
    b1 = llm.beam_search([prompt], BeamSearchParams(beam_width=1, max_tokens=5, ignore_eos=True))[0].sequences
    assert len(b1) == 1 and b1[0].tokens == prompt + greedy.token_ids
    assert abs(b1[0].cum_logprob - greedy.cumulative_logprob) < 1e-4
    b4 = llm.beam_search([prompt], BeamSearchParams(beam_width=4, max_tokens=5, ignore_eos=True))[0].sequences
    assert len(b4) == 4 and len({tuple(s.tokens) for s in b4}) == 4
    assert b4[0].cum_logprob >= b1[0].cum_logprob - 1e-5
    assert all(b4[i].cum_logprob >= b4[i + 1].cum_logprob for i in range(3))
    llm.shutdown()


def test_encode_embed_score():
    from tokenweave_b200 import LLM
    llm = LLM("tiny-llama", dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16,
              max_num_batched_tokens=64, seed=5)
    a, b = list(range(5, 45)), list(range(50, 150))      # b is prefilled in chunks
    enc = llm.encode([a, b])
    H = llm.llm_engine.config.model.hidden_size
    assert [tuple(e.data.shape) for e in enc] == [(H,), (H,)]
    emb = llm.embed([a, b])
    for e, raw in zip(emb, enc):
        assert abs(float(e.data.norm()) - 1.0) < 1e-5
        assert torch.allclose(e.data, raw.data / raw.data.norm(), atol=1e-6)
    s = llm.score(a, [a, b])
    assert abs(s[0] - 1.0) < 1e-5 and s[1] < 0.9999
    # a later generate() is unaffected by the capture switch
    assert not llm.llm_engine.core.executor.worker.runner.capture_hidden
    llm.shutdown()


def test_min_tokens_masks_eos_and_allowed_token_ids_restrict_generation():
    from tokenweave_b200 import LLM
    llm = LLM("tiny-llama", dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16,
              max_num_batched_tokens=128, seed=5)
    prompt = list(range(3, 30))
    free = llm.generate([prompt], SamplingParams(temperature=0, max_tokens=6, ignore_eos=True))[0].outputs[0].token_ids
    eos_like = free[1]                       # make the second greedy token a stop token
    early = llm.generate([prompt], SamplingParams(temperature=0, max_tokens=6, stop_token_ids=[eos_like]))[0].outputs[0]
    assert early.token_ids == free[:2] and early.finish_reason == "stop"
    late = llm.generate([prompt], SamplingParams(temperature=0, max_tokens=6, stop_token_ids=[eos_like], min_tokens=4))[0].outputs[0]
    assert len(late.token_ids) >= 4 and eos_like not in late.token_ids[:3]
    only = llm.generate([prompt], SamplingParams(temperature=0.9, seed=1, max_tokens=8, ignore_eos=True,
                                                 allowed_token_ids=[10, 11, 12]))[0].outputs[0].token_ids
    assert set(only) <= {10, 11, 12}
    llm.shutdown()


def test_guided_choice_generates_exactly_one_of_the_choices():
    from tokenweave_b200 import LLM
    llm = LLM("tiny-llama", dtype="float32", device="cpu", block_size=16, max_num_batched_tokens=128, seed=7)   # byte tokenizer
    choices = ["yes", "no", "maybe", "yes please"]
    for temp, seed in ((0.0, None), (1.0, 3), (1.0, 4), (1.5, 5)):
        out = llm.generate(["Answer:"], SamplingParams(temperature=temp, seed=seed, max_tokens=32, guided_choice=choices))[0]
        assert out.outputs[0].text in choices, out.outputs[0].text
        assert out.outputs[0].finish_reason == "stop"
    # token-id form without a tokenizer
    raw = LLM("tiny-llama", dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16,
              max_num_batched_tokens=128, seed=7)
    ids = raw.generate([[1, 2, 3]], SamplingParams(temperature=0, max_tokens=8, ignore_eos=True,
                                                   guided_choice_token_ids=[[5, 6, 7], [9, 9]]))[0].outputs[0].token_ids
    assert ids in ([5, 6, 7], [9, 9])
    llm.shutdown()
    raw.shutdown()


def test_classify_with_a_sequence_classification_checkpoint(tmp_path):
    from tokenweave_b200 import LLM
    from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
    from tokenweave_b200.models.loader import save_hf_checkpoint
    from tw_testing import hf_config_dict, make_hf_state, naive_logits
    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    st = make_hf_state(cfg, seed=8)
    head = torch.randn(3, cfg.hidden_size, generator=torch.Generator().manual_seed(1)) * 0.2
    ckpt = {k: v for k, v in st.items() if k != "lm_head.weight"}
    ckpt["score.weight"] = head
    hf = hf_config_dict(cfg)
    hf["architectures"] = ["LlamaForSequenceClassification"]
    save_hf_checkpoint(ckpt, hf, str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16,
              max_num_batched_tokens=64)
    prompts = [list(range(7, 90)), [5, 6, 7]]
    outs = llm.classify(prompts)
    for o, p in zip(outs, prompts):
        want = torch.softmax(naive_logits(cfg, {**st, "lm_head.weight": head}, p)[-1], -1)
        assert len(o.probs) == 3 and abs(sum(o.probs) - 1.0) < 1e-5
        assert torch.allclose(torch.tensor(o.probs), want, atol=1e-4)
    llm.shutdown()
    plain = LLM("tiny-llama", dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16)
    with pytest.raises(ValueError):
        plain.classify([[1, 2, 3]])
    plain.shutdown()


def test_truncate_prompt_tokens_and_priority_argument():
    llm = LLM("tiny-llama", dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16,
              max_num_batched_tokens=64, scheduling_policy="priority", max_num_seqs=1)
    long_prompt = list(range(5, 105))
    sp = SamplingParams(temperature=0, max_tokens=3, ignore_eos=True, truncate_prompt_tokens=20)
    a = llm.generate([long_prompt], sp)[0]
    b = llm.generate([long_prompt[-20:]], SamplingParams(temperature=0, max_tokens=3, ignore_eos=True))[0]
    assert a.prompt_token_ids == long_prompt[-20:] and a.outputs[0].token_ids == b.outputs[0].token_ids
    # one sequence at a time: the urgent request finishes first although it was submitted last
    outs = llm.generate([[1, 2, 3], [4, 5, 6], [7, 8, 9]], SamplingParams(temperature=0, max_tokens=2, ignore_eos=True),
                        priority=[2, 1, 0])
    t = [o.metrics.finished_time for o in outs]
    assert t[2] < t[1] < t[0]
    llm.shutdown()


def test_a_non_zero_device_status_word_stops_the_engine_before_tokens_are_emitted():
    """The runner reads the status word together with the sampled ids; a kernel that gave up on a wait must
    end the engine instead of letting tokens computed from un-reduced data through. The word is faked here
    (there is no device on this box): the second step reports a peer time-out."""
    from tokenweave_b200.engine.core import EngineDeadError
    llm = _llm()
    runner = llm.llm_engine.core.executor.worker.runner
    calls = {"n": 0}

    def fake_status():
        calls["n"] += 1
        return torch.tensor([2 if calls["n"] >= 2 else 0], dtype=torch.int32)
    runner._status_src = fake_status
    with pytest.raises(EngineDeadError, match="peer"):
        llm.generate(["abc"], SamplingParams(temperature=0, max_tokens=5, ignore_eos=True))
    assert calls["n"] == 2
    assert llm.llm_engine.core.dead
    # only the first step's token was recorded; the failed step emitted nothing
    req = next(iter(llm.llm_engine.core.scheduler.requests.values()))
    assert len(req.output_token_ids) == 1
    with pytest.raises(EngineDeadError):
        llm.generate(["abc"], SamplingParams(max_tokens=1))
    # the workers can put their communication state back collectively (a no-op for one CPU rank)
    llm.llm_engine.core.executor.collective_rpc("reset_comm_state")


def test_kv_fingerprint_keeps_models_apart(tmp_path):
    from tokenweave_b200.engine.kv_connector import KVTransferConfig, SharedStorageConnector
    cfg = KVTransferConfig(shared_storage_path=str(tmp_path))
    a = SharedStorageConnector(cfg, 0, 1, "modelA")
    b = SharedStorageConnector(cfg, 0, 1, "modelB")
    k = torch.zeros(2, 16, 1, 8)
    a.save_block(b"\x01" * 8, k, k)
    assert a.available(b"\x01" * 8) and not b.available(b"\x01" * 8)
    with pytest.raises(ValueError, match="shape"):
        a.load_block(b"\x01" * 8, (3, 16, 1, 8))
    assert a.load_block(b"\x01" * 8, (2, 16, 1, 8))[0].shape == k.shape
