"""Sampler on synthetic logits (CPU): support restriction by top-k / top-p / min-p, penalties,
seeded determinism, log-probabilities, and agreement of empirical frequencies with the softmax."""
import math

import torch

from tokenweave_b200.layers.sampler import Sampler, apply_penalties
from tokenweave_b200.sampling_params import SamplingParams


def _draw(logits_row, sp, n=4000, seed=0):
    s = Sampler()
    g = torch.Generator().manual_seed(seed)
    logits = logits_row.unsqueeze(0).repeat(n, 1)
    out = s(logits, [sp] * n, [g] * n, [[]] * n, [[]] * n)
    return out.token_ids.long()


def test_greedy_is_argmax_and_mixed_batches_keep_greedy_rows():
    torch.manual_seed(0)
    logits = torch.randn(6, 50)
    s = Sampler()
    out = s(logits, [SamplingParams(temperature=0)] * 6, [None] * 6)
    assert out.token_ids.tolist() == logits.argmax(-1).tolist()
    params = [SamplingParams(temperature=0), SamplingParams(temperature=1.0, seed=1)] * 3
    gens = [None if p.greedy else torch.Generator().manual_seed(1) for p in params]
    out = s(logits, params, gens)
    for i in (0, 2, 4):
        assert int(out.token_ids[i]) == int(logits[i].argmax())


def test_top_k_top_p_min_p_restrict_the_support():
    logits = torch.tensor([4.0, 3.0, 2.0, 1.0, 0.0, -1.0, -2.0, -3.0])
    assert set(_draw(logits, SamplingParams(top_k=3)).tolist()) <= {0, 1, 2}
    p = torch.softmax(logits, -1)
    # smallest prefix of the sorted distribution whose mass reaches 0.8
    k = int((p.cumsum(0) < 0.8).sum()) + 1
    assert set(_draw(logits, SamplingParams(top_p=0.8)).tolist()) <= set(range(k))
    keep = {i for i in range(8) if p[i] >= 0.2 * p[0]}
    assert set(_draw(logits, SamplingParams(min_p=0.2)).tolist()) <= keep
    # top_k=1 is greedy whatever the temperature
    assert set(_draw(logits, SamplingParams(top_k=1, temperature=5.0)).tolist()) == {0}


def test_frequencies_follow_the_tempered_softmax():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0])
    for temp in (1.0, 0.5):
        ids = _draw(logits, SamplingParams(temperature=temp), n=20000, seed=3)
        freq = torch.bincount(ids, minlength=4).float() / ids.numel()
        want = torch.softmax(logits / temp, -1)
        assert (freq - want).abs().max() < 0.015, (freq, want)


def test_seeded_requests_repeat_and_differ_across_seeds():
    torch.manual_seed(1)
    logits = torch.randn(1, 1000)
    s = Sampler()

    def run(seed):
        g = torch.Generator().manual_seed(seed)
        return [int(s(logits, [SamplingParams(seed=seed)], [g]).token_ids[0]) for _ in range(8)]
    assert run(7) == run(7)
    assert run(7) != run(8)


def test_penalties():
    logits = torch.tensor([[2.0, -2.0, 1.0, 0.5]])
    sp = SamplingParams(repetition_penalty=2.0)
    out = apply_penalties(logits.clone(), [sp], [[0]], [[1]])
    assert out.tolist() == [[1.0, -4.0, 1.0, 0.5]]          # seen tokens: positive halved, negative doubled
    sp = SamplingParams(presence_penalty=0.5, frequency_penalty=0.25)
    out = apply_penalties(logits.clone(), [sp], [[0]], [[2, 2, 3]])
    assert out.tolist() == [[2.0, -2.0, 1.0 - 0.5 - 0.5, 0.5 - 0.5 - 0.25]]   # prompt tokens are not counted


def test_logprobs_hold_the_sampled_token_and_the_top_n():
    torch.manual_seed(2)
    logits = torch.randn(2, 30)
    s = Sampler()
    out = s(logits, [SamplingParams(temperature=0, logprobs=3), SamplingParams(temperature=0)], [None, None])
    assert out.logprobs[1] is None
    lp = out.logprobs[0]
    ref = torch.log_softmax(logits[0], -1)
    top = ref.topk(3).indices.tolist()
    assert set(top) <= set(lp) and int(out.token_ids[0]) in lp
    for t, v in lp.items():
        assert math.isclose(v, float(ref[t]), abs_tol=1e-6)


def test_logprobs_are_the_models_own_even_when_penalties_and_masks_change_the_choice():
    logits = torch.tensor([[1.0, 5.0, 3.0, 2.0]])
    ref = torch.log_softmax(logits[0], -1)
    out = Sampler()(logits.clone(), [SamplingParams(temperature=0, logprobs=2, logit_bias={1: -100.0})], [None], [[]], [[]])
    assert int(out.token_ids[0]) == 2                      # the bias moved the choice away from token 1
    lp = out.logprobs[0]
    assert math.isclose(lp[2], float(ref[2]), abs_tol=1e-6)
    assert math.isclose(lp[1], float(ref[1]), abs_tol=1e-6)     # token 1 is still the model's most likely one


def test_logit_bias_allowed_tokens_bad_words_min_tokens():
    logits = torch.tensor([[1.0, 5.0, 3.0, 2.0, 0.0, -1.0]])
    s = Sampler()

    def pick(sp, outputs=()):
        return int(s(logits.clone(), [sp], [None], [[]], [list(outputs)]).token_ids[0])
    assert pick(SamplingParams(temperature=0)) == 1
    assert pick(SamplingParams(temperature=0, logit_bias={1: -100, "3": 10})) == 3      # string keys as in JSON bodies
    assert pick(SamplingParams(temperature=0, allowed_token_ids=[0, 4, 5])) == 0
    assert pick(SamplingParams(temperature=0, bad_words_token_ids=[[1]])) == 2           # single-token word: always banned
    assert pick(SamplingParams(temperature=0, bad_words_token_ids=[[7, 1]])) == 1        # prefix 7 not generated yet
    assert pick(SamplingParams(temperature=0, bad_words_token_ids=[[7, 1]]), outputs=[3, 7]) == 2
    # below min_tokens the EOS and stop tokens cannot be sampled
    sp = SamplingParams(temperature=0, min_tokens=3, stop_token_ids=[2], eos_token_id=1)
    assert pick(sp, outputs=[0]) == 3 and pick(sp, outputs=[0, 0, 0]) == 1
    # sampled (non-greedy) rows honour the masks too
    ids = _draw(logits[0], SamplingParams(allowed_token_ids=[2, 3]), n=500)
    assert set(ids.tolist()) <= {2, 3}
    import pytest
    with pytest.raises(ValueError):
        SamplingParams(allowed_token_ids=[])
