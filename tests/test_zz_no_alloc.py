"""The allocation-free single-query attention entry point (``tw_attn_decode_noalloc``).

Some callers of this library cannot call cudaMalloc: a process in which another framework owns all
device memory through its pool, a job held to a memory budget fixed at start-up, a serving loop that
cannot afford cudaMalloc's implicit synchronisation. For them the library exports one entry point
that keeps the split-KV partial results in a fixed 4 MiB array of its own instead of a caller-provided
workspace. This test calls it through its exported C symbol and checks it against the regular entry
point (``tw_attn_decode`` with a torch-allocated workspace) on two calls in a row, the second with
different inputs so that whatever the first call left in the shared array would show.

The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

vp, ll, i32, f32 = C.c_void_p, C.c_longlong, C.c_int, C.c_float


def _symbols():
    from tokenweave_b200.ops import _native
    lib = _native.load()
    new = lib.tw_attn_decode_noalloc
    new.restype = C.c_int
    new.argtypes = [vp, ll, vp, vp, i32, vp, ll, vp, vp, vp, i32, vp, i32, i32, i32, i32, f32, i32, vp]
    old = lib.tw_attn_decode          # argtypes already set by the package
    return lib, new, old


def _case(seed, kvs, hq, hkv, D, page):
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_blocks = sum((kv + page - 1) // page for kv in kvs) + 2
    rnd = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)
    kc, vc = rnd(n_blocks, page, hkv, D), rnd(n_blocks, page, hkv, D)
    max_blocks = max((kv + page - 1) // page for kv in kvs)
    bt = torch.zeros(len(kvs), max_blocks, dtype=torch.int32)
    cur = 1
    for b, kv in enumerate(kvs):
        n = (kv + page - 1) // page
        bt[b, :n] = torch.arange(cur, cur + n, dtype=torch.int32)
        cur += n
    q = rnd(len(kvs), hq * D)
    i32t = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    n = len(kvs)
    return q, kc, vc, bt.cuda(), i32t(list(range(n))), i32t(list(range(n))), i32t(kvs)


def _run_both(lib, new, old, seed, kvs, hq, hkv, D, page, splits):
    q, kc, vc, bt, rows, seqs, kvl = _case(seed, kvs, hq, hkv, D, page)
    n = len(kvs)
    stream = torch.cuda.current_stream().cuda_stream
    scale = D ** -0.5
    ref_out = torch.zeros_like(q)
    part_o = torch.empty(n * hq * splits * D, dtype=torch.float32, device="cuda")
    part_ml = torch.empty(n * hq * splits * 2, dtype=torch.float32, device="cuda")
    rc = old(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), page, ref_out.data_ptr(), ref_out.stride(0),
             rows.data_ptr(), seqs.data_ptr(), kvl.data_ptr(), n, bt.data_ptr(), bt.shape[1], hq, hkv, D, scale,
             splits, part_o.data_ptr(), part_ml.data_ptr(), 0, 0.0, stream)     # no sliding window, no soft cap
    assert rc == 0, lib.tw_last_error()
    out = torch.zeros_like(q)
    rc = new(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), page, out.data_ptr(), out.stride(0),
             rows.data_ptr(), seqs.data_ptr(), kvl.data_ptr(), n, bt.data_ptr(), bt.shape[1], hq, hkv, D, scale,
             splits, stream)
    assert rc == 0, lib.tw_last_error()
    torch.cuda.synchronize()
    assert ref_out.abs().max().item() > 0
    torch.testing.assert_close(out.float(), ref_out.float(), atol=2e-2, rtol=2e-2)


def test_no_alloc_matches_regular_entry_point_twice():
    lib, new, old = _symbols()
    _run_both(lib, new, old, seed=1, kvs=[700, 33, 4096, 1], hq=8, hkv=1, D=128, page=16, splits=8)
    _run_both(lib, new, old, seed=2, kvs=[129, 2000, 64], hq=16, hkv=2, D=128, page=128, splits=5)


def test_no_alloc_rejects_oversized_request():
    lib, new, _ = _symbols()
    q, kc, vc, bt, rows, seqs, kvl = _case(3, [64] * 4, 64, 8, 128, 16)
    out = torch.zeros_like(q)
    # 4 tokens x 64 heads x 64 splits x 130 floats = 8.5 MB, more than the 4 MiB the library holds
    rc = new(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), 16, out.data_ptr(), out.stride(0),
             rows.data_ptr(), seqs.data_ptr(), kvl.data_ptr(), 4, bt.data_ptr(), bt.shape[1], 64, 8, 128, 0.088,
             64, torch.cuda.current_stream().cuda_stream)
    assert rc == 1
    assert b"scratch" in lib.tw_last_error()
    torch.cuda.synchronize()
