"""Tensor-core decode attention (csrc/attn_decode_tc.cu) against the fp32 paged-attention reference and the
SIMT kernel: grouped-query shapes, ragged lengths, small pages, with and without split-KV."""
import pytest
import torch

from tokenweave_b200 import ops
from tokenweave_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"
BF = torch.bfloat16


def _paged(kvs, hkv, D, page, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    n_blocks = sum((kv + page - 1) // page for kv in kvs) + 3
    kc = torch.randn(n_blocks, page, hkv, D, generator=g).to(DEV, BF)
    vc = torch.randn(n_blocks, page, hkv, D, generator=g).to(DEV, BF)
    perm = torch.randperm(n_blocks, generator=g).tolist()
    max_blocks = max((kv + page - 1) // page for kv in kvs) + 1
    bt = torch.zeros(len(kvs), max_blocks, dtype=torch.int32)
    cur = 0
    for b, kv in enumerate(kvs):
        n = (kv + page - 1) // page
        bt[b, :n] = torch.tensor(perm[cur:cur + n], dtype=torch.int32)
        cur += n
    return kc, vc, bt.to(DEV)


@pytest.mark.parametrize("hq,hkv,page,kvs,sm_count", [
    (8, 1, 128, [300, 1000, 257, 2048, 129], 1),        # enough CTAs for the pretend machine: no split
    (8, 1, 128, [300, 1000, 257, 2048, 129], 148),      # split-KV (some splits own no tile for the short ones)
    (32, 8, 16, [700, 256, 3000], 148),                 # four query heads per KV head, 16-token pages
    (16, 1, 64, [512, 1500], 148),                      # sixteen query heads per KV head: N is full
    (6, 2, 128, [1024] * 40, 148),                      # odd group size
])
# "tcp" is the persistent form: sm_count = 1 there means ONE CTA walks every work item
@pytest.mark.parametrize("variant", ["tc", "tcp"])
def test_tc_decode_matches_reference(hq, hkv, page, kvs, sm_count, variant):
    D = 128
    kc, vc, bt = _paged(kvs, hkv, D, page, seed=len(kvs) + hq)
    T = len(kvs)
    q = (torch.randn(T, hq * D, generator=torch.Generator().manual_seed(1)) * 1.5).to(DEV, BF)
    scale = D ** -0.5
    cu = list(range(T + 1))
    expect = ref.paged_attention(q, kc, vc, cu, kvs, bt, hq, hkv, D, scale)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)         # noqa: E731
    rows, lens = i32(list(range(T))), i32(kvs)
    simt = expect.clone()
    if hq // hkv <= 8:          # the SIMT kernel serves groups of up to eight query heads
        ops.set_decode_variant("simt")
        ops.attn_decode(q, kc, vc, simt, rows, rows, lens, T, bt, hq, hkv, D, scale, max(kvs), sm_count=sm_count)
    out = torch.zeros_like(q)
    ops.set_decode_variant(variant)
    try:
        ops.attn_decode(q, kc, vc, out, rows, rows, lens, T, bt, hq, hkv, D, scale, max(kvs), sm_count=sm_count)
        torch.cuda.synchronize()
        ops.check_status()
    finally:
        ops.set_decode_variant(None)
    err = (out.float() - expect.float()).abs().max().item()
    err_simt = (simt.float() - expect.float()).abs().max().item()
    assert err < 3e-2, (err, err_simt)
