"""Engine core in a process of its own (ZMQ + msgpack boundary): same results as the in-process core, requests
and results cross the sockets, a dead core surfaces as EngineDeadError."""
import os
import signal

import pytest
import torch

from tokenweave_b200 import LLM, SamplingParams
from tokenweave_b200.engine.core import EngineDeadError
from tokenweave_b200.engine.core_client import MPEngineCoreClient, decode_request, encode_request, _pack, _unpack
from tokenweave_b200.engine.request import Request


def _llm(**kw):
    args = dict(dtype="float32", device="cpu", tokenizer="byte", block_size=16, max_num_batched_tokens=64)
    args.update(kw)
    return LLM("tiny-llama", **args)


def test_request_round_trips_through_msgpack():
    sp = SamplingParams(temperature=0.7, top_k=5, stop=["ab"], logit_bias={3: -2.0}, bad_words_token_ids=[[1, 2]],
                        guided_choice_token_ids=[[4, 5]], seed=11, logprobs=2)
    req = Request("r1", [1, 2, 3], sp, eos_token_id=2, prompt="abc", priority=3)
    back = decode_request(_unpack(_pack(encode_request(req))))
    assert (back.request_id, back.prompt_token_ids, back.eos_token_id, back.prompt, back.priority) == ("r1", [1, 2, 3], 2, "abc", 3)
    assert back.sampling_params == sp


def test_core_process_matches_the_in_process_core():
    prompts = ["hello world, this is a long enough prompt to be chunked " * 3, "abc", "the quick brown fox"]
    sp = SamplingParams(temperature=0, max_tokens=12, logprobs=2, n=1)
    local = _llm()
    want = local.generate(prompts, sp)
    want_stop = local.generate(["abcabc"], SamplingParams(temperature=0, max_tokens=30, stop=[want[1].outputs[0].text[3:6]]))
    local.shutdown()
    remote = _llm(engine_core_process=True, max_model_len=256)
    try:
        assert isinstance(remote.llm_engine.core, MPEngineCoreClient)
        got = remote.generate(prompts, sp)
        for a, b in zip(got, want):
            assert a.outputs[0].token_ids == b.outputs[0].token_ids and a.outputs[0].text == b.outputs[0].text
            assert a.outputs[0].finish_reason == b.outputs[0].finish_reason == "length"
            assert len(a.outputs[0].logprobs) == 12
            for la, lb in zip(a.outputs[0].logprobs, b.outputs[0].logprobs):
                assert set(la) == set(lb) and all(abs(la[k] - lb[k]) < 1e-5 for k in la)
            assert a.metrics.first_token_time is not None and a.metrics.finished_time is not None
        # a stop string is found on the front end and ends the request in the core
        stop = want_stop[0].outputs[0]
        got_stop = remote.generate(["abcabc"], SamplingParams(temperature=0, max_tokens=30,
                                                              stop=[want[1].outputs[0].text[3:6]]))[0].outputs[0]
        assert (got_stop.text, got_stop.finish_reason) == (stop.text, stop.finish_reason)
        # several samples per prompt, seeded: the fan-out happens before the boundary
        many = remote.generate(["xyz"], SamplingParams(temperature=1.0, seed=5, n=3, max_tokens=6))[0]
        assert len(many.outputs) == 3 and all(len(o.token_ids) == 6 for o in many.outputs)
        # utility calls reach the workers and the scheduler through the same sockets
        assert remote.collective_rpc("check_health") == [True]
        assert remote.reset_prefix_cache() in (True, False)
        # a request the scheduler refuses comes back as an aborted request, the engine lives on
        bad = remote.generate(prompt_token_ids=[list(range(5)) * 60], sampling_params=SamplingParams(max_tokens=1))[0]
        assert bad.outputs[0].finish_reason == "abort"
        assert remote.generate(["ok"], SamplingParams(temperature=0, max_tokens=2))[0].outputs[0].finish_reason == "length"
    finally:
        remote.shutdown()


def test_a_dead_core_process_is_reported():
    llm = _llm(engine_core_process=True)
    core = llm.llm_engine.core
    try:
        os.kill(core._proc.pid, signal.SIGKILL)
        core._proc.join(10)
        with pytest.raises(EngineDeadError):
            llm.generate(["abc"], SamplingParams(max_tokens=4))
        with pytest.raises(EngineDeadError):
            llm.generate(["abc"], SamplingParams(max_tokens=4))
    finally:
        llm.shutdown()
