#!/usr/bin/env python
"""Measures every (kernel, tile width) plan of the bf16 GEMM on the linear-layer shapes of the served
models and writes the best plan per (M, SM budget) to ``tokenweave_b200/gemm_configs/NVIDIA_B200.json``
(consumed by ``tokenweave_b200/ops/gemm_table.py``). Single GPU. The analogue of the reference's
``benchmarks/kernels/benchmark_moe.py --tune`` flow for its Triton MoE kernel.

    python artifact/gemm_tune.py --models llama-3.3-70b qwen2.5-72b mixtral-8x22b --tp 8 4 2 1
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import ROOT, time_us  # noqa: E402

import torch  # noqa: E402


def shapes_for(cfg, tp: int):
    """(N, K, swiglu) of every dense linear layer of one rank."""
    D = cfg.head_dim
    hq = cfg.num_q_heads // tp
    hkv = max(1, cfg.num_kv_heads // tp)
    H = cfg.hidden_size
    out = [((hq + 2 * hkv) * D, H, 0), (H, hq * D, 0)]
    if not cfg.is_moe:
        inter = cfg.intermediate_size // tp
        out += [(inter, H, 1), (H, inter, 0)]
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--models", nargs="+", default=["llama-3.3-70b", "qwen2.5-72b", "mixtral-8x22b"])
    ap.add_argument("--tp", type=int, nargs="+", default=[8, 4, 2, 1])
    ap.add_argument("--tokens", type=int, nargs="+", default=[256, 512, 1024, 2048, 3072, 4096, 6144, 8192, 16384])
    ap.add_argument("--sm-budgets", type=int, nargs="+", default=[148, 140, 132])
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--shapes", nargs="*", default=None,
                    help="restrict the run to these weight shapes, each as N,K,swiglu (e.g. 1280,8192,0)")
    ap.add_argument("--fp8", action="store_true", help="tune tw_gemm_fp8 (e4m3 operands) instead of the bf16 GEMM")
    ap.add_argument("--out", default=None, help="default: tokenweave_b200/gemm_configs/NVIDIA_B200[_fp8].json")
    args = ap.parse_args()
    if args.out is None:
        args.out = os.path.join(ROOT, "tokenweave_b200", "gemm_configs",
                                "NVIDIA_B200_fp8.json" if args.fp8 else "NVIDIA_B200.json")
    from tokenweave_b200 import ops
    from tokenweave_b200.config import resolve_model_config
    from tokenweave_b200.ops import _native
    from tokenweave_b200.ops import gemm_table
    lib = _native.load()
    gemm_table.set_enabled(False)       # candidates must run as forced, not as an older table says
    torch.cuda.set_device(0)
    todo = []
    for m in args.models:
        cfg = resolve_model_config(m)
        for tp in args.tp:
            if cfg.num_q_heads % tp:
                continue
            for s in shapes_for(cfg, tp):
                if s not in todo:
                    todo.append(s)
    if args.shapes:
        want = {tuple(int(v) for v in sh.split(",")) for sh in args.shapes}
        todo = [t for t in todo if t in want]
    table = {}
    if os.path.exists(args.out):
        with open(args.out) as f:
            table = json.load(f)
    for (N, K, sw) in todo:
        w = (torch.randn(2 * N if sw else N, K, device="cuda") * 0.02).to(torch.bfloat16)
        rows = []
        for M in args.tokens:
            if M * max(N, K) * 2 > 6 << 30:
                continue
            a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            if args.fp8:
                (aq, a_s), (wq, w_s) = ops.quant_fp8(a), ops.quant_fp8(w)
            for sms in args.sm_budgets:
                best = None
                for kernel in (2, 1):
                    # CTA pairs also have tiles wider than one MMA (plain epilogue only): 320 .. 512 columns
                    widths = (list(range(512, 63, -64)) if (kernel == 2 and not sw) else
                              range(256, 63, -64) if (kernel == 2 or sw) else range(256, 63, -32))
                    for bn in widths:
                        if args.fp8:
                            us = time_us(lambda: ops.gemm_fp8(aq, wq, a_s, w_s, out=out, swiglu=bool(sw), max_ctas=sms,
                                                              plan=kernel * 1000 + bn), warmup=2, iters=args.iters)
                        else:
                            lib.tw_gemm_set_kernel_override(kernel)
                            lib.tw_gemm_set_tile_override(bn)
                            us = time_us(lambda: ops.gemm(a, w, out=out, swiglu=bool(sw), max_ctas=sms), warmup=2,
                                         iters=args.iters)
                        # candidates run widest first; a narrower tile must win by 2 % to replace it
                        if best is None or us < best[2] * 0.98:
                            best = (kernel, bn, us)
                lib.tw_gemm_set_kernel_override(0)
                lib.tw_gemm_set_tile_override(0)
                rows.append([M, sms, best[0], best[1], round(best[2], 1)])
            del a, out
        table[f"{N},{K},{sw}"] = rows
        print(f"N={N} K={K} swiglu={sw}: " + " ".join(f"M{r[0]}/{r[1]}sm:k{r[2]}bn{r[3]}" for r in rows if r[1] == 148), flush=True)
        del w
    ops.check_status()
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    with open(args.out, "w") as f:
        json.dump(table, f, indent=0)
    print(f"wrote {args.out} ({len(table)} shapes)")


if __name__ == "__main__":
    main()
