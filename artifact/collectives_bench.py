#!/usr/bin/env python
"""In-kernel all-reduce / reduce-scatter / all-gather against NCCL, per CTA count (figures 5, 6, 7 of
the paper; reference: artifact/figure_5_6_7/bench.py:65-150).

Launch with ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 artifact/collectives_bench.py``.
Message: bf16 [T, 8192]. Columns in microseconds (median, cold L2, max over ranks); every in-kernel
result is checked against NCCL."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import NVLINK_GBS_MEASURED, RESULTS_DIR, finish_ranks, init_ranks, time_us, write_rows  # noqa: E402

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="+", default=[64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384])
    ap.add_argument("--ctas", type=int, nargs="+", default=[2, 4, 8, 16, 32])
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--transport", default="auto", choices=["auto", "multimem", "p2p"])
    ap.add_argument("--out", default=os.path.join(RESULTS_DIR, "collectives_bench"))
    args = ap.parse_args()
    if args.transport == "p2p":
        os.environ["TW_DISABLE_NVLS"] = "1"
    tp = init_ranks()
    if tp.world_size < 2:
        raise SystemExit("needs at least 2 ranks")
    from tokenweave_b200 import ops
    from tokenweave_b200.parallel.comm import TPCommunicator
    from tokenweave_b200.parallel.symm_mem import create_symmetric_buffer
    H, W, rank = args.hidden, tp.world_size, tp.rank
    buf = create_symmetric_buffer(max(args.tokens), H, torch.bfloat16, tp)
    comm = TPCommunicator(buf, tp, wait_budget_ms=5000)
    g = torch.Generator(device="cuda").manual_seed(2000 + rank)
    rows = []
    for T in args.tokens:
        if T % W:
            continue
        x = (torch.rand(T, H, device="cuda", generator=g) * 2 - 1).mul_((rank + 1) / (3 * W)).to(torch.bfloat16)
        view = buf.tensor[:T]
        n = T * H // W

        def refill():
            view.copy_(x)

        ref_ar = x.clone()
        dist.all_reduce(ref_ar)
        refill()
        torch.cuda.synchronize(); dist.barrier()
        comm.all_reduce_(view, 8)
        torch.cuda.synchronize()
        ok = torch.allclose(view.float(), ref_ar.float(), atol=4e-2, rtol=4e-2)
        kw = dict(warmup=args.warmup, iters=args.iters, before=refill, sync_ranks=False)
        rs_out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        row = {"tokens": T, "world": W, "transport": "multimem" if comm.use_mc else "peer", "correct": ok,
               "nccl_ar": time_us(lambda: dist.all_reduce(view), **kw),
               "nccl_rs": time_us(lambda: dist.reduce_scatter_tensor(rs_out, view.view(-1)), **kw),
               "nccl_ag": time_us(lambda: dist.all_gather_into_tensor(view.view(-1), rs_out), **kw)}
        for c in args.ctas:
            row[f"ar_{c}"] = time_us(lambda: comm.all_reduce_(view, c), **kw)
            row[f"rs_{c}"] = time_us(lambda: comm.reduce_scatter_(view, c), **kw)
            row[f"ag_{c}"] = time_us(lambda: comm.all_gather_(view, c), **kw)
        small = torch.empty_like(x)
        row["oneshot_ar"] = time_us(lambda: comm.oneshot_all_reduce(view, small), **kw) if T * H * 2 <= (8 << 20) else None
        for op in ("ar", "rs", "ag"):
            row[f"{op}_best"] = min(row[f"{op}_{c}"] for c in args.ctas)
        row["ar_roofline_us"] = T * H * 2 / (NVLINK_GBS_MEASURED * 1e9) * 1e6
        rows.append(row)
        if rank == 0:
            print({k: (round(v, 1) if isinstance(v, float) else v) for k, v in row.items()}, flush=True)
    ops.check_status()
    if rank == 0:
        write_rows(args.out, f"collectives_w{W}", rows)
    finish_ranks()


if __name__ == "__main__":
    main()
