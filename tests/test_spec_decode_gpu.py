"""Speculative decoding on the GPU: verification steps run the drafts as a multi-token query through the
prefill attention kernel. In bf16 the verified path and the one-token decode path are different kernels,
so agreement with plain greedy decoding is checked on the leading tokens, not demanded bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(spec):
    from tokenweave_b200 import LLM, SamplingParams, ops
    llm = LLM("tiny-llama-d128", device="cuda", skip_tokenizer_init=True, max_num_batched_tokens=1024, block_size=128,
              num_gpu_blocks_override=64, seed=0, speculative_config=spec)
    g = torch.Generator().manual_seed(0)
    base = torch.randint(0, 2048, (24,), generator=g).tolist()
    prompts = [base * 6, (base[:5] * 30)[:140], torch.randint(0, 2048, (200,), generator=g).tolist()]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=32, ignore_eos=True))
    torch.cuda.synchronize()
    ops.check_status()
    sched = llm.llm_engine.core.scheduler
    stats = (sched._step, sched.num_draft_tokens, sched.num_accepted_tokens)
    toks = [o.outputs[0].token_ids for o in outs]
    llm.shutdown()
    return toks, stats


def test_speculative_decoding_runs_and_tracks_greedy():
    plain, (steps0, d0, a0) = _run(None)
    spec, (steps1, d1, a1) = _run({"method": "ngram", "num_speculative_tokens": 4})
    assert d0 == 0 and d1 > 0 and 0 < a1 <= d1
    assert all(len(t) == 32 for t in spec)
    assert steps1 < steps0
    agree = [next((i for i, (x, y) in enumerate(zip(a, b)) if x != y), len(a)) for a, b in zip(plain, spec)]
    assert sum(agree) >= 32, f"speculative and plain greedy outputs diverge too early: {agree}"
