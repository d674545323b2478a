"""Decode attention: the SIMT split-KV kernel against the tensor-core kernel, over batch / context shapes.

    python artifact/decode_attn_bench.py [--csv NAME]

Per shape: median of 8 launches timed with CUDA events after 3 warm-up launches, a 256 MB buffer written
between launches to flush L2, the K and V bytes of the batch divided by the time as achieved bandwidth, and
the largest difference between the two kernels' outputs. One GPU.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tokenweave_b200 import ops  # noqa: E402

DEV, BF = "cuda", torch.bfloat16
SHAPES = [  # batch, keys per sequence, query heads, KV heads (per rank), page
    (256, 2048, 8, 1, 128), (64, 8192, 8, 1, 128), (256, 512, 8, 1, 128), (16, 32768, 8, 1, 128),
    (192, 1100, 8, 1, 128), (256, 2048, 32, 8, 16),
]


def run_case(B, kv, hq, hkv, page, variants=("simt", "tc"), D=128):
    mb = (kv + page - 1) // page
    nb = B * mb + 2
    kc = torch.randn(nb, page, hkv, D, device=DEV, dtype=BF)
    vc = torch.randn_like(kc)
    bt = (torch.randperm(nb - 1, device=DEV)[: B * mb] + 1).to(torch.int32).view(B, mb)
    q = torch.randn(B, hq * D, device=DEV, dtype=BF)
    rows = torch.arange(B, dtype=torch.int32, device=DEV)
    lens = torch.full((B,), kv, dtype=torch.int32, device=DEV)
    out = torch.zeros_like(q)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    res, first = {}, None
    for var in variants:
        ops.set_decode_variant(var)
        launch = lambda: ops.attn_decode(q, kc, vc, out, rows, rows, lens, B, bt, hq, hkv, D, D ** -0.5, kv)  # noqa: E731
        for _ in range(3):
            launch()
        ts = []
        for _ in range(8):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            launch()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        res[var] = sorted(ts)[len(ts) // 2]
        if first is None:
            first = out.clone()
    ops.set_decode_variant(None)
    ops.check_status()
    kv_bytes = 2 * B * kv * hkv * D * 2
    row = dict(batch=B, kv_len=kv, q_heads=hq, kv_heads=hkv, page=page)
    for var in variants:
        row[var + "_us"] = round(res[var], 1)
        row[var + "_tb_s"] = round(kv_bytes / res[var] / 1e6, 2)
    row["speedup"] = round(res[variants[0]] / res[variants[-1]], 2)        # first variant over last
    row["max_abs_diff"] = float((out.float() - first.float()).abs().max())
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--csv", default=None, help="also write the rows to <results dir>/<NAME>.csv")
    ap.add_argument("--variants", default="simt,tc",
                    help="kernels to time, in order: simt, tc (one CTA per work item), tcp (persistent CTAs)")
    ns = ap.parse_args()
    variants = tuple(ns.variants.split(","))
    rows = [run_case(*s, variants=variants) for s in SHAPES]
    for r in rows:
        print(json.dumps(r), flush=True)
    if ns.csv:
        from common import RESULTS_DIR, write_rows
        write_rows(RESULTS_DIR, ns.csv, rows)


if __name__ == "__main__":
    main()
