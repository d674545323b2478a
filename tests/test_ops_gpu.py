"""CUDA kernels against the fp32 PyTorch references of the same ops."""
import math

import pytest
import torch

from tokenweave_b200 import ops
from tokenweave_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(BF)


def close(a, b, atol=2e-2, rtol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    bound = atol + rtol * b.abs()
    bad = (err > bound).sum().item()
    assert bad == 0, f"{bad}/{a.numel()} elements off, max err {err.max().item():.4g} (ref max {b.abs().max().item():.4g})"


@pytest.fixture(autouse=True)
def _status_clean():
    ops.reset_status()
    yield
    ops.check_status()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 128), (300, 1280, 1024), (1000, 1000, 200),
                                   (4096, 7168, 1024), (77, 8, 512), (2048, 8192, 3584)])
def test_gemm_plain(M, N, K):
    a, w = rnd(M, K), rnd(N, K, scale=1 / math.sqrt(K))
    out = ops.gemm(a, w)
    close(out, ref.gemm(a, w))


@pytest.mark.parametrize("bn", [320, 384, 448, 512])
@pytest.mark.parametrize("M,N,K,max_ctas", [(4096, 1280, 1024, 0), (1000, 1280, 512, 0), (512, 1000, 256, 6), (300, 640, 1088, 0)])
def test_gemm_pair_wide_tiles(M, N, K, max_ctas, bn):
    """CTA-pair kernel with tiles wider than one MMA (two MMAs per k-step, one accumulator), bias included."""
    from tokenweave_b200.ops import _native, gemm_table
    lib = _native.load()
    a, w, bias = rnd(M, K), rnd(N, K, scale=1 / math.sqrt(K)), rnd(N)
    gemm_table.set_enabled(False)
    lib.tw_gemm_set_kernel_override(2)
    lib.tw_gemm_set_tile_override(bn)
    try:
        out = ops.gemm(a, w, bias=bias, max_ctas=max_ctas)
        torch.cuda.synchronize()
    finally:
        lib.tw_gemm_set_kernel_override(0)
        lib.tw_gemm_set_tile_override(0)
        gemm_table.set_enabled(True)
    close(out, ref.gemm(a, w, bias))


def test_gemm_bias_rowscale_strided_out():
    M, N, K = 513, 1280, 1024
    a, w, bias = rnd(M, K), rnd(N, K, scale=1 / math.sqrt(K)), rnd(N)
    rs = torch.rand(M, device=DEV)
    big = torch.zeros(M, N + 64, device=DEV, dtype=BF)
    out = big[:, 32:32 + N]
    ops.gemm(a, w, out=out, bias=bias, row_scale=rs)
    close(out, ref.gemm(a, w, bias, rs))
    assert big[:, :32].abs().max().item() == 0 and big[:, 32 + N:].abs().max().item() == 0


def test_gemm_strided_a():
    M, N, K = 256, 512, 256
    big = rnd(M, 3 * K)
    a = big[:, K:2 * K]
    w = rnd(N, K, scale=1 / math.sqrt(K))
    close(ops.gemm(a, w), ref.gemm(a.contiguous(), w))


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (300, 3584, 1024), (1000, 200, 256), (4096, 3696, 512)])
def test_gemm_swiglu(M, I, K):
    a, w = rnd(M, K), rnd(2 * I, K, scale=1 / math.sqrt(K))
    out = ops.gemm(a, w, swiglu=True)
    assert out.shape == (M, I)
    close(out, ref.gemm_swiglu(a, w))


def test_gemm_max_ctas():
    M, N, K = 2048, 2048, 512
    a, w = rnd(M, K), rnd(N, K, scale=1 / math.sqrt(K))
    close(ops.gemm(a, w, max_ctas=7), ref.gemm(a, w))


@pytest.mark.parametrize("T,H", [(7, 256), (83, 8192), (1000, 6144), (64, 4096)])
def test_norms(T, H):
    x, r, w = rnd(T, H), rnd(T, H), (1 + 0.1 * torch.randn(H, device=DEV)).to(BF)
    close(ops.rmsnorm(x, w, 1e-5), ref.rmsnorm(x, w, 1e-5))
    x1, r1 = x.clone(), r.clone()
    x2, r2 = x.clone(), r.clone()
    ops.add_rmsnorm_(x1, r1, w, 1e-5)
    ref.add_rmsnorm_(x2, r2, w, 1e-5)
    close(x1, x2)
    assert torch.equal(r1, r2)
    x1, x2 = x.clone(), x.clone()
    ro1, ro2 = torch.empty_like(x), torch.empty_like(x)
    ops.rmsnorm_copy_(x1, ro1, w, 1e-5, max_ctas=5)
    ref.rmsnorm_copy_(x2, ro2, w, 1e-5)
    close(x1, x2)
    assert torch.equal(ro1, ro2)


@pytest.mark.parametrize("hq,hkv,D,page", [(8, 2, 128, 16), (64, 8, 128, 128), (4, 2, 64, 32)])
def test_rope_kv_write(hq, hkv, D, page):
    T, blocks = 333, 40
    qkv = rnd(T + 5, (hq + 2 * hkv) * D)
    pos = torch.randint(0, 4000, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(blocks * page, device=DEV)[:T].to(torch.int32)
    slots[5] = -1
    cs = ref.build_cos_sin_cache(D, 4096, 500000.0, device=DEV)
    kc, vc = torch.zeros(blocks, page, hkv, D, device=DEV, dtype=BF), torch.zeros(blocks, page, hkv, D, device=DEV, dtype=BF)
    kc2, vc2 = kc.clone(), vc.clone()
    q1, q2 = qkv.clone(), qkv.clone()
    ops.rope_kv_write_(q1, pos, slots, cs, kc, vc, hq, hkv, D, write_k_back=True)
    ref.rope_kv_write_(q2[:T], pos, slots, cs, kc2, vc2, hq, hkv, D)
    close(q1, q2, atol=1e-2)
    close(kc, kc2, atol=1e-2)
    assert torch.equal(vc, vc2)


@pytest.mark.parametrize("hq,hkv,D", [(8, 2, 128), (5, 1, 64), (2, 2, 256)])
def test_rope_kv_write_with_qk_norm(hq, hkv, D):
    """Per-head RMSNorm of q and k inside the rope + cache-write launch (Qwen3 layout)."""
    T, blocks, page = 77, 8, 16
    qkv = rnd(T, (hq + 2 * hkv) * D) * 3
    pos = torch.randint(0, 4000, (T,), device=DEV, dtype=torch.int32)
    slots = torch.randperm(blocks * page, device=DEV)[:T].to(torch.int32)
    cs = ref.build_cos_sin_cache(D, 4096, 1e6, device=DEV)
    qw, kw = (1 + 0.3 * torch.randn(D, device=DEV)).to(BF), (1 + 0.3 * torch.randn(D, device=DEV)).to(BF)
    kc, vc = torch.zeros(blocks, page, hkv, D, device=DEV, dtype=BF), torch.zeros(blocks, page, hkv, D, device=DEV, dtype=BF)
    kc2, vc2 = kc.clone(), vc.clone()
    q1, q2 = qkv.clone(), qkv.clone()
    ops.rope_kv_write_(q1, pos, slots, cs, kc, vc, hq, hkv, D, write_k_back=True, qk_norm=(qw, kw, 1e-6))
    ref.rope_kv_write_(q2, pos, slots, cs, kc2, vc2, hq, hkv, D, qk_norm=(qw, kw, 1e-6))
    close(q1, q2, atol=3e-2)
    close(kc, kc2, atol=3e-2)
    assert torch.equal(vc, vc2)
    # and against the unrounded fp32 definition: normalise, scale, rotate
    x = qkv[:, : (hq + hkv) * D].float().view(T, hq + hkv, D)
    w = torch.cat([qw.float().expand(hq, D), kw.float().expand(hkv, D)], 0)
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    c, s = cs[pos.long(), : D // 2].unsqueeze(1), cs[pos.long(), D // 2:].unsqueeze(1)
    want = torch.cat([x[..., : D // 2] * c - x[..., D // 2:] * s, x[..., D // 2:] * c + x[..., : D // 2] * s], -1)
    close(q1[:, : (hq + hkv) * D].float().view(T, hq + hkv, D), want, atol=6e-2)


def test_swiglu_embedding_argmax():
    x = rnd(300, 2 * 3584)
    close(ops.swiglu(x), ref.swiglu(x))
    table = rnd(1000, 512)
    ids = torch.randint(0, 2000, (257,), device=DEV, dtype=torch.int32)
    out = ops.embedding(ids, table, vocab_start=500, vocab_end=1500)
    assert torch.equal(out, ref.embedding(ids, table, 500, 1500))
    logits = torch.randn(33, 128256, device=DEV)
    assert torch.equal(ops.argmax(logits).long(), torch.argmax(logits, -1))


def _make_paged(seqs, hkv, D, page, extra_blocks=3):
    """seqs: list of (q_len, kv_len). Returns caches filled with random data + metadata."""
    n_blocks = sum((kv + page - 1) // page for _, kv in seqs) + extra_blocks
    kc, vc = rnd(n_blocks, page, hkv, D), rnd(n_blocks, page, hkv, D)
    perm = torch.randperm(n_blocks).tolist()
    max_blocks = max((kv + page - 1) // page for _, kv in seqs) + 1
    bt = torch.zeros(len(seqs), max_blocks, dtype=torch.int32)
    cur = 0
    for b, (_, kv) in enumerate(seqs):
        n = (kv + page - 1) // page
        bt[b, :n] = torch.tensor(perm[cur:cur + n], dtype=torch.int32)
        cur += n
    cu = [0]
    for ql, _ in seqs:
        cu.append(cu[-1] + ql)
    return kc, vc, bt.to(DEV), cu, [kv for _, kv in seqs]


@pytest.mark.parametrize("hq,hkv,D,page,seqs", [
    (4, 2, 128, 16, [(128, 128)]),
    (8, 1, 128, 128, [(300, 300), (17, 17), (129, 129)]),
    (8, 2, 128, 16, [(200, 1000), (1, 77), (128, 640), (5, 5)]),
    (4, 4, 64, 32, [(333, 333), (64, 500)]),
    (16, 2, 128, 64, [(1024, 1024), (700, 2048)]),
    (4, 2, 64, 32, [(333, 333), (64, 500), (1, 130)]),
    (6, 1, 128, 128, [(513, 1300)]),
])
# one head per CTA / two heads of a KV group per CTA / persistent CTAs with the key range split between the
# softmax groups (on every SM, and on 3 CTAs so that each walks several items in both directions)
@pytest.mark.parametrize("variant", [1, 2, 3, (3, 3)])
def test_attn_prefill(hq, hkv, D, page, seqs, variant):
    from tokenweave_b200.ops import _native
    variant, max_ctas = variant if isinstance(variant, tuple) else (variant, 0)
    _native.load().tw_attn_set_variant(variant)
    kc, vc, bt, cu, kv_lens = _make_paged(seqs, hkv, D, page)
    T = cu[-1]
    q = rnd(T, hq * D)
    scale = D ** -0.5
    expect = ref.paged_attention(q, kc, vc, cu, kv_lens, bt, hq, hkv, D, scale)
    tile_seq, tile_q0 = [], []
    for b, (ql, _) in enumerate(seqs):
        for q0 in range(0, ql, 128):
            tile_seq.append(b)
            tile_q0.append(q0)
    out = torch.zeros_like(q)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    try:
        ops.attn_prefill(q, kc, vc, out, i32(cu), i32(kv_lens), bt, i32(tile_seq), i32(tile_q0), len(tile_seq), hq,
                         hkv, D, scale, max_ctas=max_ctas)
        torch.cuda.synchronize()
        ops.check_status()
    finally:
        _native.load().tw_attn_set_variant(-1)
    close(out, expect, atol=2e-2, rtol=3e-2)


@pytest.mark.parametrize("window,softcap", [(200, 0.0), (0, 7.5), (77, 30.0), (5000, 0.0)])
@pytest.mark.parametrize("hq,hkv,D,page,seqs", [
    (8, 2, 128, 16, [(200, 1000), (1, 77), (128, 640), (5, 5)]),
    (4, 4, 64, 32, [(333, 333), (64, 500)]),
    (16, 2, 128, 128, [(1024, 1024), (700, 2048)]),
])
def test_attn_sliding_window_and_softcap(hq, hkv, D, page, seqs, window, softcap):
    """Prefill tiles and single-query tokens under a sliding window and / or a soft cap on the scores."""
    kc, vc, bt, cu, kv_lens = _make_paged(seqs, hkv, D, page)
    T = cu[-1]
    q = rnd(T, hq * D, scale=2.0)
    scale = D ** -0.5
    expect = ref.paged_attention(q, kc, vc, cu, kv_lens, bt, hq, hkv, D, scale, window=window, softcap=softcap)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    tile_seq, tile_q0, tok_row, tok_seq, tok_kv = [], [], [], [], []
    for b, (ql, kv) in enumerate(seqs):
        if ql >= 16:
            for q0 in range(0, ql, 128):
                tile_seq.append(b)
                tile_q0.append(q0)
        else:
            for i in range(ql):
                tok_row.append(cu[b] + i)
                tok_seq.append(b)
                tok_kv.append(kv - ql + i + 1)
    out = torch.zeros_like(q)
    ops.attn_prefill(q, kc, vc, out, i32(cu), i32(kv_lens), bt, i32(tile_seq), i32(tile_q0), len(tile_seq), hq, hkv, D,
                     scale, window=window, softcap=softcap)
    if tok_row:
        ops.attn_decode(q, kc, vc, out, i32(tok_row), i32(tok_seq), i32(tok_kv), len(tok_row), bt, hq, hkv, D, scale,
                        max(tok_kv), window=window, softcap=softcap)
    torch.cuda.synchronize()
    ops.check_status()
    close(out, expect, atol=2e-2, rtol=3e-2)
    # every row as a single-query token through the decode kernel (split-KV included)
    rows = list(range(T))
    seq_of = [b for b, (ql, _) in enumerate(seqs) for _ in range(ql)]
    kv_of = [kv - ql + i + 1 for (ql, kv) in seqs for i in range(ql)]
    out2 = torch.zeros_like(q)
    ops.attn_decode(q, kc, vc, out2, i32(rows), i32(seq_of), i32(kv_of), T, bt, hq, hkv, D, scale, max(kv_of),
                    window=window, softcap=softcap)
    torch.cuda.synchronize()
    close(out2, expect, atol=2e-2, rtol=3e-2)


@pytest.mark.parametrize("hq,hkv,D,page,kvs", [
    (8, 1, 128, 16, [1, 31, 32, 33, 700]),
    (64, 8, 128, 128, [5000, 77]),
    (6, 1, 128, 64, [300] * 40),
    (4, 2, 64, 16, [129, 4096]),
])
@pytest.mark.parametrize("variant", ["simt", None])     # None: the library's choice (tensor cores where they apply)
def test_attn_decode(hq, hkv, D, page, kvs, variant):
    ops.set_decode_variant(variant)
    seqs = [(1, kv) for kv in kvs]
    kc, vc, bt, cu, kv_lens = _make_paged(seqs, hkv, D, page)
    T = len(kvs)
    q = rnd(T, hq * D)
    scale = D ** -0.5
    expect = ref.paged_attention(q, kc, vc, cu, kv_lens, bt, hq, hkv, D, scale)
    out = torch.zeros_like(q)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    try:
        ops.attn_decode(q, kc, vc, out, i32(list(range(T))), i32(list(range(T))), i32(kv_lens), T, bt, hq, hkv, D,
                        scale, max(kvs))
        torch.cuda.synchronize()
    finally:
        ops.set_decode_variant(None)
    close(out, expect, atol=2e-2, rtol=3e-2)


@pytest.mark.parametrize("T,H,I,E", [(64, 512, 256, 8), (1000, 1024, 512, 8), (300, 6144, 2048, 8)])
def test_moe_pipeline(T, H, I, E):
    topk = 2
    x = rnd(T, H)
    gate = rnd(E, H, scale=1 / math.sqrt(H))
    w13 = rnd(E, 2 * I, H, scale=1 / math.sqrt(H))
    w2 = rnd(E, H, I, scale=1 / math.sqrt(I))
    tw, ids, logits = ops.moe_router(x, gate, topk, want_logits=True)
    rw, rids, rlogits = ref.moe_router(x, gate, topk)
    close(logits, rlogits, atol=1e-2)
    # top-k ids may differ only where probabilities are nearly tied
    same = (ids.long() == rids.long()).all(dim=-1)
    assert same.float().mean().item() > 0.98
    close(tw[same], rw[same], atol=1e-3)
    expect = ref.moe_experts(x, w13, w2, tw, ids)

    n_pairs = T * topk
    max_rows = n_pairs + E * 127
    max_tiles = (max_rows + 127) // 128
    i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=DEV)
    offs, cursor, tile_expert, meta = i32(E + 1), i32(E), i32(max_tiles), i32(2)
    ops.moe_align(ids, E, 128, offs, cursor, tile_expert, meta)
    a_sorted = torch.zeros(max_tiles * 128, H, device=DEV, dtype=BF)
    row_scale = torch.zeros(max_tiles * 128, device=DEV)
    sorted_pos = i32(T, topk)
    ops.moe_scatter(x, ids, tw, offs, cursor, a_sorted, row_scale, sorted_pos, E)
    counts = torch.bincount(ids.flatten().long(), minlength=E)
    padded = ((counts + 127) // 128 * 128)
    assert meta[1].item() == padded.sum().item() and meta[0].item() == padded.sum().item() // 128
    act = ops.gemm(a_sorted, w13.view(E * 2 * I, H), swiglu=True, tile_expert=tile_expert, num_m_tiles=meta[:1],
                   n_per_expert=2 * I)
    y = ops.gemm(act, w2.view(E * H, I), row_scale=row_scale, tile_expert=tile_expert, num_m_tiles=meta[:1],
                 n_per_expert=H)
    out = torch.empty(T, H, device=DEV, dtype=BF)
    ops.moe_combine(y, sorted_pos, out, topk)
    close(out, expect, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("kind", sorted(ref.ACTIVATION_KINDS))
def test_activations(kind):
    gated = ref.ACTIVATION_KINDS[kind] <= 4
    x = rnd(333, 2 * 1096 if gated else 1096, scale=2.0)
    out = ops.activation(x, kind, param=0.25)
    close(out, ref.activation(x, kind, 0.25))
    # strided input: a column slice of a wider buffer
    wide = rnd(64, 4096, scale=2.0)
    view = wide[:, 512:512 + (1024 if gated else 512)]
    close(ops.activation(view, kind, param=0.25), ref.activation(view, kind, 0.25))


def test_copy_and_swap_pages():
    cache = rnd(24, 16, 2, 128)
    want = cache.clone()
    pairs = torch.tensor([[0, 5], [1, 6], [7, 23], [3, 2]], dtype=torch.int64, device=DEV)
    for s, d in pairs.tolist():
        want[d] = cache[s]
    ops.copy_pages(cache, pairs)
    assert torch.equal(cache, want)
    host = torch.zeros(10, 16, 2, 128, dtype=BF).pin_memory()
    out_pairs = [(4, 0), (5, 1), (6, 2), (20, 7)]
    ops.swap_pages(cache, host, out_pairs)
    torch.cuda.synchronize()
    for s, d in out_pairs:
        assert torch.equal(host[d], cache[s].cpu())
    back = torch.zeros_like(cache)
    ops.swap_pages(host, back, [(0, 9), (1, 10), (7, 3)])
    torch.cuda.synchronize()
    assert torch.equal(back[9], cache[4]) and torch.equal(back[10], cache[5]) and torch.equal(back[3], cache[20])


@pytest.mark.parametrize("T,H,D", [(1, 4, 128), (77, 8, 128), (300, 3, 64)])
def test_merge_attn_states(T, H, D):
    a, b = rnd(T, H, D), rnd(T, H, D)
    la = torch.randn(H, T, device=DEV) * 3
    lb = torch.randn(H, T, device=DEV) * 3
    lb[0, 0] = -math.inf                 # an empty partial result takes weight zero
    if T > 2:
        la[1, 2] = math.inf
    out, lse = ops.merge_attn_states(a, la, b, lb, want_lse=True)
    want, want_lse = ref.merge_attn_states(a, la, b, lb)
    close(out, want)
    assert torch.allclose(lse, want_lse, atol=1e-4, rtol=1e-4)
    # against attention itself: softmax over the union of two key sets
    q = torch.randn(H, D, device=DEV)
    k = torch.randn(H, 40, D, device=DEV)
    v = torch.randn(H, 40, D, device=DEV)
    s = torch.einsum("hd,hkd->hk", q, k)
    full = torch.einsum("hk,hkd->hd", torch.softmax(s, -1), v)
    o1 = torch.einsum("hk,hkd->hd", torch.softmax(s[:, :15], -1), v[:, :15]).to(BF).unsqueeze(0).contiguous()
    o2 = torch.einsum("hk,hkd->hd", torch.softmax(s[:, 15:], -1), v[:, 15:]).to(BF).unsqueeze(0).contiguous()
    l1 = torch.logsumexp(s[:, :15], -1).unsqueeze(1).contiguous()
    l2 = torch.logsumexp(s[:, 15:], -1).unsqueeze(1).contiguous()
    close(ops.merge_attn_states(o1, l1, o2, l2)[0], full, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("T,H", [(1, 128), (77, 1024), (300, 8192), (9, 12288)])
def test_quant_fp8(T, H):
    x = rnd(T, H, scale=3.0)
    q, s = ops.quant_fp8(x)
    # The oracle runs on the CPU: torch's CUDA division by the Python scalar 448 multiplies by a reciprocal,
    # which moves the scale by an ulp and with it the 0.6 % of bf16 inputs that sit on e4m3 rounding ties.
    q_ref, s_ref = ref.quant_fp8(x.cpu())
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    static = torch.tensor([0.05], device=DEV)
    q2, _ = ops.quant_fp8(x, scale=static)
    assert torch.equal(q2.cpu().view(torch.uint8), ref.quant_fp8(x.cpu(), static.cpu())[0].view(torch.uint8))
    # fused with RMSNorm, with and without the residual add
    w = rnd(H, scale=0.5)
    qn, sn = ops.rmsnorm_quant_fp8(x, w, 1e-5)
    y = ref.rmsnorm(x, w, 1e-5)
    close(qn.float() * sn[:, None], y, atol=0.05 * y.float().abs().max().item(), rtol=0.07)
    res = rnd(T, H)
    res_want = (x + res)
    res_in = res.clone()
    qa, sa = ops.rmsnorm_quant_fp8(x, w, 1e-5, residual=res_in)
    assert torch.equal(res_in, res_want)
    y2 = ref.rmsnorm(res_want, w, 1e-5)
    close(qa.float() * sa[:, None], y2, atol=0.05 * y2.float().abs().max().item(), rtol=0.07)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 1280, 1024), (1000, 1000, 208), (4096, 7168, 1024),
                                   (77, 8, 512), (2048, 8192, 3584)])
# the library's choice / single-CTA tiles / CTA pairs, 256 and 128 columns wide / CTA pairs, wide tile
@pytest.mark.parametrize("plan", [0, 1256, 2256, 2128, 2384])
def test_gemm_fp8(M, N, K, plan):
    a, w = rnd(M, K), rnd(N, K, scale=1 / math.sqrt(K))
    aq, a_s = ops.quant_fp8(a)
    wq, w_s = ops.quant_fp8(w)
    bias = rnd(N)
    out = ops.gemm_fp8(aq, wq, a_s, w_s, bias=bias, plan=plan)
    # exact products of the same quantised operands: only accumulation order and the final rounding differ
    close(out, ref.gemm_fp8(aq, wq, a_s, w_s, bias))
    # and the quantised result approximates the bf16 product
    full = ref.gemm(a, w).float() + bias.float()
    assert (out.float() - full).abs().mean() < 0.05 * full.abs().mean() + 0.02
    # unscaled: sums of products of up to 448 * 448 that cancel; the absolute slack follows the magnitude
    raw = ref.gemm_fp8(aq, wq, None, None)
    close(ops.gemm_fp8(aq, wq, None, None, plan=plan), raw, atol=1e-4 * raw.float().abs().max().item(), rtol=2e-2)


@pytest.mark.parametrize("M,I,K", [(256, 512, 256), (1000, 3584, 1024), (4096, 3584, 8192)])
@pytest.mark.parametrize("plan", [0, 1256, 2256, 2192])
def test_gemm_fp8_swiglu(M, I, K, plan):
    a, w = rnd(M, K), rnd(2 * I, K, scale=1 / math.sqrt(K))
    aq, a_s = ops.quant_fp8(a)
    wq, w_s = ops.quant_fp8(w)
    out = ops.gemm_fp8(aq, wq, a_s, w_s, swiglu=True, plan=plan)
    assert out.shape == (M, I)
    close(out, ref.gemm_fp8(aq, wq, a_s, w_s, swiglu=True))


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 1280, 1024), (1000, 1000, 208), (4096, 7168, 1024),
                                   (77, 8, 512), (2048, 8192, 3584)])
@pytest.mark.parametrize("plan", [0, 2256, 2128, 2384])
def test_gemm_int8(M, N, K, plan):
    """int8 operands on the tensor cores (32-bit integer accumulation): exact against the integer product."""
    a, w = rnd(M, K), rnd(N, K, scale=1 / math.sqrt(K))
    aq, a_s = ops.quant_int8(a)
    wq, w_s = ops.quant_int8(w)
    bias = rnd(N)
    out = ops.gemm_int8(aq, wq, a_s, w_s, bias=bias, plan=plan)
    close(out, ref.gemm_int8(aq, wq, a_s, w_s, bias))
    full = ref.gemm(a, w).float() + bias.float()
    assert (out.float() - full).abs().mean() < 0.03 * full.abs().mean() + 0.02
    # unscaled: the integer sums themselves, exact up to the final rounding to bf16
    raw = ref.gemm_int8(aq, wq, None, None)
    got = ops.gemm_int8(aq, wq, None, None, plan=plan)
    assert torch.equal(got, raw)


@pytest.mark.parametrize("M,I,K", [(256, 512, 256), (1000, 3584, 1024)])
@pytest.mark.parametrize("plan", [0, 2256, 2192])
def test_gemm_int8_swiglu(M, I, K, plan):
    a, w = rnd(M, K), rnd(2 * I, K, scale=1 / math.sqrt(K))
    aq, a_s = ops.quant_int8(a)
    wq, w_s = ops.quant_int8(w)
    out = ops.gemm_int8(aq, wq, a_s, w_s, swiglu=True, plan=plan)
    assert out.shape == (M, I)
    close(out, ref.gemm_int8(aq, wq, a_s, w_s, swiglu=True))


@pytest.mark.parametrize("T,H", [(7, 64), (300, 8192), (33, 5120)])
def test_int8_quant_and_fused_norm(T, H):
    x = rnd(T, H, scale=3.0)
    q, s = ops.quant_int8(x)
    q_ref, s_ref = ref.quant_int8(x)
    torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
    assert (q.int() - q_ref.int()).abs().max().item() <= 1 and (q != q_ref).float().mean().item() < 1e-3
    static = torch.tensor([0.05], device=DEV)
    q2, _ = ops.quant_int8(x, static)
    assert (q2.int() - ref.quant_int8(x, static)[0].int()).abs().max().item() <= 1
    w = rnd(H, scale=0.1) + 1
    res = rnd(T, H)
    res2 = res.clone()
    q3, s3 = ops.rmsnorm_quant_int8(x, w, 1e-5, residual=res2)
    summed = x + res
    assert torch.equal(res2, summed)
    y = ref.rmsnorm(summed, w, 1e-5)
    q3_ref, s3_ref = ref.quant_int8(y)
    torch.testing.assert_close(s3, s3_ref, rtol=2e-2, atol=1e-6)
    assert (q3.int() - q3_ref.int()).abs().max().item() <= 2


def test_gather_cache_convert_fp8_permute_cols():
    seqs = [(1, 300), (1, 17), (1, 128), (1, 1)]
    hkv, D, page = 2, 128, 16
    kc, _, bt, _, kv_lens = _make_paged(seqs, hkv, D, page)
    cu = torch.tensor([0] + list(torch.tensor(kv_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    got = ops.gather_cache(kc, bt, cu, sum(kv_lens))
    assert torch.equal(got, ref.gather_cache(kc, bt, kv_lens))
    # bf16 -> e4m3 -> bf16 with a scale: what an fp8 KV cache stores and returns
    x = rnd(64, 16, hkv, D)
    f8 = ops.convert_fp8(x, scale=0.5)
    assert f8.dtype == torch.float8_e4m3fn
    want = (x.float() / 0.5).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert (f8.float() - want.float()).abs().max().item() <= 0.07 * want.float().abs().max().item()
    back = ops.convert_fp8(f8, scale=0.5)
    torch.testing.assert_close(back.float(), f8.float() * 0.5, rtol=1e-2, atol=1e-3)
    torch.testing.assert_close(back.float(), x.float(), rtol=0.07, atol=0.03)
    # column permutation
    m = rnd(37, 1000)
    perm = torch.randperm(1000, device=DEV).to(torch.int32)
    assert torch.equal(ops.permute_cols(m, perm), m[:, perm.long()])


@pytest.mark.parametrize("T,pair", [(4096, True), (4096, False), (5000, True), (300, True)])
def test_moe_layer_grouped_gemm_on_cta_pairs(T, pair):
    """The MoE layer end to end: with enough rows per expert the groups are padded to 256 rows and the grouped
    GEMMs run on CTA pairs; both forms must agree with the loop-over-experts reference."""
    from tokenweave_b200.layers.moe import FusedMoE
    from tokenweave_b200.parallel.state import set_single_process
    set_single_process(torch.device(DEV))
    H, I, E = 1024, 512, 8
    moe = FusedMoE(E, 2, H, I, dtype=BF, device=DEV)
    moe.pair_tiles = pair
    moe.gate.data.copy_(rnd(E, H, scale=1 / math.sqrt(H)))
    moe.w13.data.copy_(rnd(E, 2 * I, H, scale=1 / math.sqrt(H)))
    moe.w2.data.copy_(rnd(E, H, I, scale=1 / math.sqrt(I)))
    x = rnd(T, H)
    out = moe(x)
    torch.cuda.synchronize()
    tw, ids, _ = ops.moe_router(x, moe.gate, 2)
    want = ref.moe_experts(x, moe.w13, moe.w2, tw, ids)
    close(out, want, atol=3e-2, rtol=3e-2)
