"""Speculative decoding with n-gram drafts: the proposer, the acceptance rule, and the engine end to end
(token-for-token equal to plain greedy decoding, fewer steps on repetitive text)."""
import pytest
import torch

from tokenweave_b200 import LLM, SamplingParams
from tokenweave_b200.engine.spec_decode import SpecDecodeConfig, accept_greedy, clamp_drafts, ngram_propose


def test_ngram_proposer():
    ids = [1, 2, 3, 4, 5, 9, 9, 1, 2, 3]
    assert ngram_propose(ids, 3, max_n=3, min_n=2) == [4, 5, 9]          # suffix (1,2,3) seen at the start
    assert ngram_propose(ids, 2, max_n=3, min_n=2) == [4, 5]
    assert ngram_propose([1, 2, 3, 4], 3) == []                           # nothing repeats
    assert ngram_propose([7, 8, 7, 8, 7, 8], 4, max_n=2, min_n=2) == [7, 8]   # most recent earlier occurrence
    assert ngram_propose([5, 5], 3, max_n=4, min_n=2) == []
    assert ngram_propose([3, 1, 4, 1], 2, max_n=4, min_n=1) == [4, 1]     # falls back to the 1-gram "1"


def test_acceptance_rule_and_clamping():
    assert accept_greedy([4, 5, 6], [4, 5, 6, 7]) == [4, 5, 6, 7]        # all confirmed + the bonus token
    assert accept_greedy([4, 5, 6], [4, 9, 6, 7]) == [4, 9]              # first disagreement replaces the draft
    assert accept_greedy([4], [8, 1]) == [8]
    assert accept_greedy([], [3]) == [3]
    assert clamp_drafts([1, 2, 3, 4], num_tokens=10, max_model_len=13, max_tokens=None, num_output_tokens=0) == [1, 2]
    assert clamp_drafts([1, 2, 3, 4], 10, 100, max_tokens=6, num_output_tokens=4) == [1]
    assert clamp_drafts([1, 2, 3, 4], 10, 100, max_tokens=5, num_output_tokens=4) == []
    cfg = SpecDecodeConfig.from_user({"method": "ngram", "num_speculative_tokens": 4, "prompt_lookup_max": 5})
    assert cfg.enabled and cfg.prompt_lookup_max == 5 and cfg.prompt_lookup_min == 2
    assert not SpecDecodeConfig.from_user(None).enabled and SpecDecodeConfig.from_user(3).num_speculative_tokens == 3
    with pytest.raises(ValueError):
        SpecDecodeConfig.from_user({"method": "eagle", "num_speculative_tokens": 2})


def _engine(**kw):
    args = dict(dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=256, seed=2)
    args.update(kw)
    return LLM("tiny-llama", **args)


def _steps(llm):
    return llm.llm_engine.core.scheduler._step


def test_speculative_greedy_equals_plain_greedy_and_takes_fewer_steps():
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, 1024, (24,), generator=g).tolist()
    prompts = [base * 4, torch.randint(0, 1024, (50,), generator=g).tolist(), (base[:7] * 9)[:60]]
    sp = SamplingParams(temperature=0, max_tokens=40, ignore_eos=True)
    plain = _engine()
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    plain_steps = _steps(plain)
    plain.shutdown()
    spec = _engine(speculative_config={"method": "ngram", "num_speculative_tokens": 4, "prompt_lookup_max": 4})
    got = [o.outputs[0].token_ids for o in spec.generate(prompts, sp)]
    sched = spec.llm_engine.core.scheduler
    assert got == want
    assert all(len(t) == 40 for t in got)
    assert sched.num_draft_tokens > 0 and 0 < sched.num_accepted_tokens <= sched.num_draft_tokens
    assert _steps(spec) < plain_steps, (_steps(spec), plain_steps)
    # sampled (non-greedy) requests are not drafted for and still work next to greedy ones
    mixed = spec.generate(prompts[:2], [sp, SamplingParams(temperature=1.0, seed=1, max_tokens=12, ignore_eos=True)])
    assert mixed[0].outputs[0].token_ids == want[0] and len(mixed[1].outputs[0].token_ids) == 12
    spec.shutdown()


def test_speculative_respects_stop_token_and_limits():
    g = torch.Generator().manual_seed(1)
    base = torch.randint(0, 1024, (16,), generator=g).tolist()
    prompt = base * 5
    plain = _engine()
    ref = plain.generate([prompt], SamplingParams(temperature=0, max_tokens=30, ignore_eos=True))[0].outputs[0].token_ids
    plain.shutdown()
    stop_tok = ref[17]
    first = ref.index(stop_tok)
    spec = _engine(speculative_config=5, max_model_len=len(prompt) + 64)
    out = spec.generate([prompt], SamplingParams(temperature=0, max_tokens=30, ignore_eos=True, stop_token_ids=[stop_tok]))[0]
    assert out.outputs[0].token_ids == ref[:first + 1] and out.outputs[0].finish_reason == "stop"
    out = spec.generate([prompt], SamplingParams(temperature=0, max_tokens=7, ignore_eos=True))[0]
    assert out.outputs[0].token_ids == ref[:7] and out.outputs[0].finish_reason == "length"
    # prefix caching and chunked prefill keep working with drafts in flight
    spec2 = _engine(speculative_config=3, enable_prefix_caching=True, max_num_batched_tokens=48)
    a = spec2.generate([prompt, prompt], SamplingParams(temperature=0, max_tokens=20, ignore_eos=True))
    assert a[0].outputs[0].token_ids == ref[:20] and a[1].outputs[0].token_ids == ref[:20]
    spec.shutdown()
    spec2.shutdown()
