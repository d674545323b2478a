"""CPU paths of the small ops (activations, page copy / swap, partial-attention merge)."""
import math

import torch

from tokenweave_b200 import ops
from tokenweave_b200.ops import reference as ref


def test_activation_cpu_matches_torch():
    x = torch.randn(5, 32)
    assert torch.allclose(ops.activation(x, "gelu_and_mul"), torch.nn.functional.gelu(x[:, :16]) * x[:, 16:], atol=1e-6)
    assert torch.allclose(ops.activation(x, "quick_gelu"), x * torch.sigmoid(1.702 * x), atol=1e-6)
    assert ops.activation(x, "fatrelu_and_mul", param=0.5).shape == (5, 16)


def test_pages_cpu():
    cache = torch.arange(6 * 4, dtype=torch.float32).reshape(6, 4)
    ops.copy_pages(cache, torch.tensor([[0, 3], [1, 4]]))
    assert torch.equal(cache[3], cache[0]) and torch.equal(cache[4], cache[1])
    dst = torch.zeros(3, 4)
    ops.swap_pages(cache, dst, [(5, 0), (2, 2)])
    assert torch.equal(dst[0], cache[5]) and torch.equal(dst[2], cache[2]) and dst[1].abs().sum() == 0


def test_merge_cpu_is_exact_softmax_merge():
    H, D = 2, 8
    q, k, v = torch.randn(H, D), torch.randn(H, 12, D), torch.randn(H, 12, D)
    s = torch.einsum("hd,hkd->hk", q, k)
    full = torch.einsum("hk,hkd->hd", torch.softmax(s, -1), v)
    parts = []
    for sl in (slice(0, 5), slice(5, 12)):
        parts.append((torch.einsum("hk,hkd->hd", torch.softmax(s[:, sl], -1), v[:, sl]).unsqueeze(0),
                      torch.logsumexp(s[:, sl], -1).unsqueeze(1)))
    out, lse = ref.merge_attn_states(parts[0][0], parts[0][1], parts[1][0], parts[1][1])
    assert torch.allclose(out[0], full, atol=1e-5)
    assert torch.allclose(lse[:, 0], torch.logsumexp(s, -1), atol=1e-5)
    empty = torch.full((H, 1), -math.inf)
    out2, _ = ref.merge_attn_states(parts[0][0], parts[0][1], parts[1][0], empty)
    assert torch.allclose(out2, parts[0][0], atol=1e-6)
