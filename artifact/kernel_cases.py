#!/usr/bin/env python
"""Runs ONE kernel on a small, fixed case a few times: the command to put under ``ncu`` (single GPU).

    python artifact/kernel_cases.py gemm --m 4096 --n 8192 --k 4096
    ncu --set full --clock-control none -k regex:gemm_bf16 -s 2 -c 2 -o results/gemm python artifact/kernel_cases.py gemm

Inputs are larger than the 126 MB L2 where the kernel's real workloads are, but stay within a few GB.
Prints the CUDA-event time of the last launch and the achieved rate against the measured peaks."""
from __future__ import annotations

import argparse
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import measured_peaks  # noqa: E402

import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "gemm_swiglu", "gemm_fp8", "rmsnorm_quant_fp8", "attn_prefill", "attn_decode", "add_rmsnorm", "rope_kv",
                                     "moe_router", "moe_layer", "fused_local", "gemm_rs_norm_local", "ag_gemm_local",
                                     "sample"])
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--attn-variant", type=int, default=-1,
                    help="attn_prefill: -1 library default, 0 auto, 1 one head per CTA, 2 head pairs, 3 persistent with split key range")
    ap.add_argument("--q-tokens", type=int, default=0,
                    help="attn_prefill: only the last N tokens are queries (a chunk of a longer prompt, or the second "
                         "token subset of the overlap schedule); 0 = all")
    ap.add_argument("--max-ctas", type=int, default=0, help="attn_prefill variant 3: SM budget (0 = all)")
    ap.add_argument("--attn-ring", type=int, default=0, help="attn_prefill head pairs: K/V tile slots (0 = all that fit)")
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--decode-variant", default=None, choices=["simt", "tc", "tcp"],
                    help="attn_decode: SIMT kernel (attn_decode_kernel), tensor cores (attn_decode_tc_kernel) or their "
                         "persistent form; default: the library's choice")
    args = ap.parse_args()
    from tokenweave_b200 import ops
    from tokenweave_b200.ops import _native
    _native.load().tw_attn_set_variant(args.attn_variant)
    if args.decode_variant:
        ops.set_decode_variant(args.decode_variant)
    _native.load().tw_attn_set_ring(args.attn_ring)
    torch.cuda.set_device(0)
    dev, BF = "cuda", torch.bfloat16
    peaks = measured_peaks()
    flops = bytes_moved = 0

    if args.case == "sample":
        B, V = 256, 128256          # a full decode batch over the Llama-3 vocabulary: 131 MB of fp32 logits
        logits = torch.randn(B, V, device=dev) * 3
        packed = ops.pack_sample_params([0.8] * B, [50] * B, [0.9] * B, [0.0] * B, range(B)).to(dev)
        fn = lambda: ops.sample(logits, packed)
        bytes_moved = B * V * 4 * 11          # the row is read 11 times (max, 4 + sum + 4 radix passes, draw), mostly from L2
    elif args.case in ("gemm", "gemm_swiglu"):
        M, N, K = args.m, args.n, args.k
        a = torch.randn(M, K, device=dev).to(BF)
        sw = args.case == "gemm_swiglu"
        w = (torch.randn(2 * N if sw else N, K, device=dev) / math.sqrt(K)).to(BF)
        out = torch.empty(M, N, device=dev, dtype=BF)
        fn = lambda: ops.gemm(a, w, out=out, swiglu=sw)
        flops = 2 * M * (2 * N if sw else N) * K
    elif args.case == "gemm_fp8":
        M, N, K = args.m, args.n, args.k
        aq, a_s = ops.quant_fp8(torch.randn(M, K, device=dev).to(BF))
        wq, w_s = ops.quant_fp8((torch.randn(N, K, device=dev) / math.sqrt(K)).to(BF))
        out = torch.empty(M, N, device=dev, dtype=BF)
        fn = lambda: ops.gemm_fp8(aq, wq, a_s, w_s, out=out)
        flops = 2 * M * N * K
    elif args.case == "rmsnorm_quant_fp8":
        T, H = args.tokens, args.hidden
        x, r = torch.randn(T, H, device=dev).to(BF), torch.randn(T, H, device=dev).to(BF)
        w = torch.ones(H, device=dev, dtype=BF)
        q = torch.empty(T, H, device=dev, dtype=torch.float8_e4m3fn)
        fn = lambda: ops.rmsnorm_quant_fp8(x, w, 1e-5, residual=r, out=q)
        bytes_moved = T * H * (2 + 2 + 2 + 1)
    elif args.case == "attn_prefill":
        T, hq, hkv, D, page = args.tokens, args.heads, args.kv_heads, args.head_dim, 128
        nb = T // page + 1
        kc, vc = torch.randn(nb, page, hkv, D, device=dev).to(BF), torch.randn(nb, page, hkv, D, device=dev).to(BF)
        Tq = args.q_tokens or T
        q = torch.randn(Tq, hq * D, device=dev).to(BF)
        out = torch.empty_like(q)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        tiles = list(range(0, Tq, 128))[::-1]
        meta = (i32([0, Tq]), i32([T]), torch.arange(nb, dtype=torch.int32, device=dev).view(1, -1), i32([0] * len(tiles)), i32(tiles))
        fn = lambda: ops.attn_prefill(q, kc, vc, out, meta[0], meta[1], meta[2], meta[3], meta[4], len(tiles), hq, hkv, D, D ** -0.5,
                                      max_ctas=args.max_ctas)
        flops = 4 * hq * D * (T * T - (T - Tq) * (T - Tq)) // 2
    elif args.case == "attn_decode":
        B, kv, hq, hkv, D, page = 256, 2048, args.heads, args.kv_heads, 128, 128
        nb = B * (kv // page) + 1
        kc, vc = torch.randn(nb, page, hkv, D, device=dev).to(BF), torch.randn(nb, page, hkv, D, device=dev).to(BF)
        q = torch.randn(B, hq * D, device=dev).to(BF)
        out = torch.empty_like(q)
        bt = (torch.arange(B * (kv // page), dtype=torch.int32, device=dev) + 1).view(B, -1)
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        kvl = torch.full((B,), kv, dtype=torch.int32, device=dev)
        fn = lambda: ops.attn_decode(q, kc, vc, out, ar, ar, kvl, B, bt, hq, hkv, D, D ** -0.5, kv)
        bytes_moved = 2 * B * kv * hkv * D * 2
    elif args.case == "add_rmsnorm":
        T, H = args.tokens, args.hidden
        x, r = torch.randn(T, H, device=dev).to(BF), torch.randn(T, H, device=dev).to(BF)
        w = torch.ones(H, device=dev, dtype=BF)
        fn = lambda: ops.add_rmsnorm_(x, r, w, 1e-5)
        bytes_moved = 4 * T * H * 2
    elif args.case == "rope_kv":
        from tokenweave_b200.ops import reference as ref
        T, hq, hkv, D, page = args.tokens, args.heads, args.kv_heads, 128, 128
        qkv = torch.randn(T, (hq + 2 * hkv) * D, device=dev).to(BF)
        kc = torch.zeros(T // page + 1, page, hkv, D, device=dev, dtype=BF)
        vc = torch.zeros_like(kc)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        cs = ref.build_cos_sin_cache(D, T, 500000.0, device=dev)
        fn = lambda: ops.rope_kv_write_(qkv, pos, pos, cs, kc, vc, hq, hkv, D)
        bytes_moved = T * (2 * hq + 4 * hkv) * D * 2
    elif args.case == "moe_router":
        T, H = args.tokens, 6144
        x = torch.randn(T, H, device=dev).to(BF)
        g = (torch.randn(8, H, device=dev) / math.sqrt(H)).to(BF)
        fn = lambda: ops.moe_router(x, g, 2)
        bytes_moved = T * H * 2
    elif args.case == "moe_layer":
        # one Mixtral-8x22B MoE layer as a GPU of an 8-way tensor-parallel group sees it: 8 experts, top-2,
        # hidden 6144, 2048 intermediate columns per expert; router, align, scatter, two grouped GEMMs, combine
        from tokenweave_b200.layers.moe import FusedMoE
        from tokenweave_b200.parallel.state import set_single_process
        set_single_process(torch.device(dev))
        T, H, I, E = args.tokens, 6144, 2048, 8
        moe = FusedMoE(E, 2, H, I, dtype=BF, device=dev)
        moe.gate.data.copy_(torch.randn(E, H, device=dev) / math.sqrt(H))
        moe.w13.data.copy_(torch.randn(E, 2 * I, H, device=dev) / math.sqrt(H))
        moe.w2.data.copy_(torch.randn(E, H, I, device=dev) / math.sqrt(I))
        x = torch.randn(T, H, device=dev).to(BF)
        out = torch.empty_like(x)
        fn = lambda: moe(x, out=out)
        flops = 2 * (2 * T) * H * (3 * I)
    elif args.case in ("gemm_rs_norm_local", "ag_gemm_local"):
        # the GEMM fused with its collective on one GPU acting as a world of one (peer transport): the GEMM CTAs
        # and the communication CTAs run as on several GPUs, the "peers" are this GPU's own buffer
        from tokenweave_b200.ops import _native
        T, H, K = args.m, args.hidden, args.k
        flags = torch.zeros(1024, dtype=torch.int32, device=dev)
        flagp = torch.tensor([flags.data_ptr()], dtype=torch.int64, device=dev)
        w_norm = torch.ones(H, device=dev, dtype=BF)
        stream = torch.cuda.current_stream().cuda_stream
        if args.case == "gemm_rs_norm_local":      # o_proj / down_proj: [T, K] x [H, K]^T -> reduce-scatter -> norm
            a = torch.randn(T, K, device=dev).to(BF)
            w = (torch.randn(H, K, device=dev) / math.sqrt(K)).to(BF)
            rows, res = torch.zeros(T, H, device=dev, dtype=BF), torch.randn(T, H, device=dev).to(BF)
            bases = torch.tensor([rows.data_ptr()], dtype=torch.int64, device=dev)
            fn = lambda: _native.call("tw_gemm_rs_norm", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), T, H, K,
                                      None, rows.data_ptr(), None, bases.data_ptr(), flagp.data_ptr(), 0, 1, 10 ** 9,
                                      ops.status_word().data_ptr(), 0, T, res.data_ptr(), res.stride(0),
                                      w_norm.data_ptr(), 1e-5, 16, 0, stream)
            flops = 2 * T * H * K
        else:                                      # qkv_proj / gate_up_proj: all-gather -> [T, H] x [N, H]^T
            N = args.n
            rows = torch.randn(T, H, device=dev).to(BF)
            w = (torch.randn(N, H, device=dev) / math.sqrt(H)).to(BF)
            c = torch.empty(T, N, device=dev, dtype=BF)
            bases = torch.tensor([rows.data_ptr()], dtype=torch.int64, device=dev)
            epoch = torch.zeros(2, dtype=torch.int32, device=dev)
            fn = lambda: _native.call("tw_ag_gemm", rows.data_ptr(), w.data_ptr(), w.stride(0), N, c.data_ptr(),
                                      c.stride(0), None, T, N, H, 0, 0, None, bases.data_ptr(), flagp.data_ptr(),
                                      epoch.data_ptr(), 0, 1, 10 ** 9, ops.status_word().data_ptr(), 0, T, 16, 0,
                                      stream)
            flops = 2 * T * N * H
    else:   # fused_local: the fused collective kernel on one GPU acting as a world of one (peer transport)
        from tokenweave_b200.ops import _native
        T, H = args.tokens, args.hidden
        x, r = torch.randn(T, H, device=dev).to(BF), torch.randn(T, H, device=dev).to(BF)
        w = torch.ones(H, device=dev, dtype=BF)
        pads = torch.zeros(4096, dtype=torch.int32, device=dev)
        bases = torch.tensor([x.data_ptr()], dtype=torch.int64, device=dev)
        padp = torch.tensor([pads.data_ptr()], dtype=torch.int64, device=dev)
        fn = lambda: _native.call("tw_fused_rs_norm_ag", None, bases.data_ptr(), padp.data_ptr(), 0, 1, 0, 10 ** 9,
                                  ops.status_word().data_ptr(), 0, r.data_ptr(), r.stride(0), w.data_ptr(), T, H,
                                  1e-5, 16, 0, 0, torch.cuda.current_stream().cuda_stream)
        bytes_moved = 4 * T * H * 2

    ms = 0.0
    for _ in range(args.launches):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e)
    ops.check_status()
    line = f"{args.case}: {ms * 1e3:.1f} us"
    if flops:
        tf = flops / ms / 1e9
        line += f", {tf:.0f} TFLOP/s = {tf / peaks['bf16_tflops']:.2f} of {peaks['source']} cuBLAS burst peak"
    if bytes_moved:
        gbs = bytes_moved / ms / 1e6
        line += f", {gbs:.0f} GB/s = {gbs / peaks['hbm_gbs']:.2f} of {peaks['source']} copy bandwidth"
    print(line)


if __name__ == "__main__":
    main()
