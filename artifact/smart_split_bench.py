#!/usr/bin/env python
"""Cost of cutting the MLP block's GEMMs in two ("smart split", figure 9 of the paper; reference:
artifact/figure_9/bench.py:63-133): time of gate_up(+SwiGLU) -> down on M tokens unsplit versus on
(M/2 + offset) and (M/2 - offset) tokens back to back, for offsets 0..256. Single GPU; shapes are one
rank's share of Llama-3.3-70B at the given TP size."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import RESULTS_DIR, time_us, write_rows  # noqa: E402

import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--tokens", type=int, nargs="+", default=[1024, 1536, 2048, 2560, 3072, 3584, 4096, 8192])
    ap.add_argument("--offsets", type=int, nargs="+", default=[0, 64, 128, 192, 256])
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--intermediate", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--out", default=os.path.join(RESULTS_DIR, "smart_split"))
    args = ap.parse_args()
    from tokenweave_b200 import ops
    torch.cuda.set_device(0)
    H, I = args.hidden, args.intermediate // args.tp
    w13 = (torch.randn(2 * I, H, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(H, I, device="cuda") * 0.02).to(torch.bfloat16)
    rows = []
    for M in args.tokens:
        x = torch.randn(M, H, device="cuda").to(torch.bfloat16)
        act = torch.empty(M, I, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)

        def mlp(lo, hi):
            ops.gemm(x[lo:hi], w13, out=act[lo:hi], swiglu=True)
            ops.gemm(act[lo:hi], w2, out=out[lo:hi])

        row = {"tokens": M, "tp": args.tp, "unsplit_us": time_us(lambda: mlp(0, M), iters=args.iters)}
        for off in args.offsets:
            cut = M // 2 + off
            row[f"split_off{off}_us"] = time_us(lambda: (mlp(0, cut), mlp(cut, M)), iters=args.iters)
        rows.append(row)
        print({k: (round(v, 1) if isinstance(v, float) else v) for k, v in row.items()}, flush=True)
    ops.check_status()
    write_rows(args.out, f"smart_split_tp{args.tp}", rows)


if __name__ == "__main__":
    main()
