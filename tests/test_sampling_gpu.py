"""Fused sampling kernel against the sort-based PyTorch sampler: identical support under top-k / top-p /
min-p, frequencies that follow the tempered softmax, greedy rows, exact repeatability of a seed."""
import pytest
import torch

from tokenweave_b200 import ops
from tokenweave_b200.layers.sampler import Sampler, _filter_top_k_top_p
from tokenweave_b200.sampling_params import SamplingParams

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sample_many(row, temperature, top_k, top_p, min_p, n, seed0=1):
    logits = row.to(DEV).unsqueeze(0).repeat(n, 1).contiguous()
    packed = ops.pack_sample_params([temperature] * n, [top_k] * n, [top_p] * n, [min_p] * n,
                                    [seed0 * 7919 + i for i in range(n)])
    return ops.sample(logits, packed.to(DEV)).long().cpu()


def _allowed(row, temperature, top_k, top_p, min_p):
    V = row.numel()
    x = (row / temperature).unsqueeze(0)
    k = torch.tensor([V if top_k <= 0 else min(top_k, V)])
    masked = _filter_top_k_top_p(x.clone(), k, torch.tensor([top_p]), torch.tensor([min_p]))
    return masked[0], set(torch.isfinite(masked[0]).nonzero().flatten().tolist())


@pytest.mark.parametrize("V", [50, 1000, 128256])
@pytest.mark.parametrize("temperature,top_k,top_p,min_p", [(1.0, -1, 1.0, 0.0), (0.7, 5, 1.0, 0.0), (1.0, -1, 0.6, 0.0),
                                                           (1.3, 40, 0.9, 0.0), (1.0, -1, 1.0, 0.05), (0.9, 7, 0.5, 0.02)])
def test_support_and_frequencies_match_the_sort_based_sampler(V, temperature, top_k, top_p, min_p):
    g = torch.Generator().manual_seed(V + top_k)
    row = torch.randn(V, generator=g) * 2.5
    masked, allowed = _allowed(row, temperature, top_k, top_p, min_p)
    ids = _sample_many(row, temperature, top_k, top_p, min_p, n=6000)
    got = set(ids.tolist())
    assert got <= allowed, f"sampled outside the support: {sorted(got - allowed)[:5]}"
    want = torch.softmax(masked, -1)
    freq = torch.bincount(ids, minlength=V).float() / ids.numel()
    # the heaviest tokens are hit with the right frequency (3.5 sigma of a binomial with 6000 draws)
    top = want.topk(min(5, len(allowed))).indices
    for t in top.tolist():
        sigma = (want[t] * (1 - want[t]) / ids.numel()).sqrt().item()
        assert abs(freq[t].item() - want[t].item()) < 3.5 * sigma + 2e-3, (t, freq[t].item(), want[t].item())
    if len(allowed) > 1 and want.max() < 0.999:
        assert len(got) > 1


def test_greedy_rows_seeds_and_mixed_batches():
    torch.manual_seed(0)
    logits = (torch.randn(64, 32000) * 3).to(DEV)
    greedy = ops.sample(logits, ops.pack_sample_params([0.0] * 64, [-1] * 64, [1.0] * 64, [0.0] * 64, range(64)).to(DEV))
    assert torch.equal(greedy.long(), logits.argmax(-1))
    p = ops.pack_sample_params([1.0] * 64, [50] * 64, [0.95] * 64, [0.0] * 64, [11] * 64).to(DEV)
    a, b = ops.sample(logits, p), ops.sample(logits, p)
    assert torch.equal(a, b)
    p2 = ops.pack_sample_params([1.0] * 64, [50] * 64, [0.95] * 64, [0.0] * 64, [12] * 64).to(DEV)
    assert not torch.equal(a, ops.sample(logits, p2))
    # through the Sampler: greedy rows of a mixed batch stay greedy, seeded rows repeat
    params = [SamplingParams(temperature=0), SamplingParams(temperature=1.0, seed=3, top_p=0.9)] * 32
    s = Sampler(seed=0)
    o1 = s(logits, params, [None] * 64, [[]] * 64, [[1, 2]] * 64).token_ids
    o2 = Sampler(seed=99)(logits, params, [None] * 64, [[]] * 64, [[1, 2]] * 64).token_ids
    assert torch.equal(o1[0::2].long(), logits[0::2].argmax(-1))
    assert torch.equal(o1[1::2], o2[1::2])
    o3 = s(logits, params, [None] * 64, [[]] * 64, [[1, 2, 3]] * 64).token_ids       # next position: new draws
    assert not torch.equal(o1[1::2], o3[1::2])
