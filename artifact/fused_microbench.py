#!/usr/bin/env python
"""Fused all-reduce + residual-add + RMSNorm microbenchmark (figures 4 and 10 of the paper;
reference: artifact/figure_4_10/bench.py:63-237).

Launch: ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 artifact/fused_microbench.py``.
Per rank: a bf16 partial-sum tensor [T, 8192] and residual [T, 8192] ~ N(0,1), RMSNorm weight ~ N(1, 0.1),
eps 1e-5, seed per rank. Columns (microseconds, median, cold L2, max over ranks):

  norm_full      add+RMSNorm on all T rows (what follows an unfused all-reduce)
  norm_shard     add+RMSNorm on this rank's T/N rows
  nccl_ar        NCCL all-reduce
  nccl_ar_norm   NCCL all-reduce + add+RMSNorm (the baseline the fused kernel replaces)
  mm_ar / mm_rs / mm_ag   in-kernel all-reduce / reduce-scatter / all-gather
  simple_fusion  RS, norm, AG as three phases of one kernel
  fused[c]       the product kernel on c CTAs, c in --ctas ("fused_best" = min over c)
  roofline_us    T*H*2 bytes over the measured 770 GB/s per direction; frac = roofline / fused_best
  ref_*          with --reference-kernels: the reference's OWN kernels (csrc/tokenweave_fused_kernels.cu and
                 csrc/tokenweave_artifact_kernels.cu, unchanged, built by baseline/build_ref_kernels.py) on the same
                 box, same inputs, same timing loop, driven as artifact/figure_4_10/bench.py:136-160 drives them:
                 ref_fused[c] / ref_fused_best (fused_rs_ln_ag_cta), ref_mm_ar (multimem_ar_cta),
                 ref_simple_fusion (simple_fusion_rs_ln_ag_cta)
Each fused result is checked against NCCL all-reduce + reference RMSNorm with atol = rtol = 4e-2.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import NVLINK_GBS_MEASURED, RESULTS_DIR, finish_ranks, init_ranks, time_us, write_rows  # noqa: E402

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def burst_us(fn, n: int, reps: int = 9) -> float:
    """Per-launch device time of ``n`` back-to-back launches (median over ``reps``, max over ranks)."""
    import statistics
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) * 1e3 / n)
    med = statistics.median(times)
    if dist.is_initialized():
        t = torch.tensor([med], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        med = float(t.item())
    return med


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="+", default=[64, 256, 1024, 4096, 8192, 16384])
    ap.add_argument("--ctas", type=int, nargs="+", default=[2, 4, 8, 16, 32])
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--transport", default="auto", choices=["auto", "multimem", "p2p"])
    ap.add_argument("--sync-ranks", action="store_true", help="host barrier before every timed iteration")
    ap.add_argument("--burst", type=int, default=20,
                    help="also time this many back-to-back launches per event pair (steady-state latency per launch, "
                         "warm L2, no host in between: how the kernels run inside a model step); 0 disables")
    ap.add_argument("--reference-kernels", action="store_true",
                    help="also time the reference's own kernels from baseline/_ref/tw_ref_kernels (their device waits "
                         "have no bound: they run only after this build's kernel passed on every rank for the same T)")
    ap.add_argument("--out", default=os.path.join(RESULTS_DIR, "fused_microbench"))
    args = ap.parse_args()
    if args.transport == "p2p":
        os.environ["TW_DISABLE_NVLS"] = "1"
    tp = init_ranks()
    from tokenweave_b200 import ops
    from tokenweave_b200.ops import reference as ref
    from tokenweave_b200.parallel.comm import TPCommunicator
    from tokenweave_b200.parallel.symm_mem import create_symmetric_buffer

    H, W, rank = args.hidden, tp.world_size, tp.rank
    Tmax = max(args.tokens)
    buf = create_symmetric_buffer(Tmax, H, torch.bfloat16, tp)
    ref_ops = ref_buf = None
    if args.reference_kernels and W > 1:
        lib = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref",
                           "tw_ref_kernels", "tw_ref_kernels.so")
        if not os.path.exists(lib):
            raise SystemExit(f"{lib} is missing: run python baseline/build_ref_kernels.py first")
        torch.ops.load_library(lib)
        ref_ops = torch.ops.tw_ref
        # a symmetric buffer of its own, through PyTorch's rendezvous as the reference does (llama.py:437-441)
        ref_buf = create_symmetric_buffer(Tmax, H, torch.bfloat16, tp, provider="torch")
        if not ref_buf.has_multicast:
            raise SystemExit("the reference's kernels need the NVLS multicast mapping")
    comm = TPCommunicator(buf, tp, wait_budget_ms=5000)
    g = torch.Generator(device="cuda").manual_seed(1000 + rank)
    gw = torch.Generator(device="cuda").manual_seed(7)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=gw)).to(torch.bfloat16)
    rows = []
    for T in args.tokens:
        if T % W:
            continue
        x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
        res0 = torch.randn(T, H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).to(torch.bfloat16)
        res = res0.clone()
        view = buf.tensor[:T]
        scratch = torch.empty_like(x)
        rpr = T // W

        def refill():
            view.copy_(x)

        # correctness of the product kernel for this T
        xs = x.float()
        if W > 1:
            dist.all_reduce(xs)
        expect_res = xs.to(torch.bfloat16) + res0
        expect = ref.rmsnorm(expect_res, w, 1e-5)
        refill()
        res.copy_(res0)
        torch.cuda.synchronize()
        if W > 1:
            dist.barrier()
        comm.fused_allreduce_add_rmsnorm_(view, res, w, 1e-5, max_ctas=16)
        torch.cuda.synchronize()
        ok = torch.allclose(view.float(), expect.float(), atol=4e-2, rtol=4e-2)
        if W > 1:
            flag = torch.tensor([int(ok)], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(flag.item())

        row = {"tokens": T, "hidden": H, "world": W, "transport": "multimem" if comm.use_mc else ("peer" if comm.in_kernel else "local"),
               "correct": ok}
        # No host barrier between iterations (the reference does none either): every timed kernel
        # synchronises the ranks itself, so they stay in step, and a host barrier would add its own exit
        # skew (10+ us) to the small-message latencies.
        kw = dict(warmup=args.warmup, iters=args.iters, before=refill, sync_ranks=args.sync_ranks)
        row["norm_full"] = time_us(lambda: ops.add_rmsnorm_(scratch, res, w, 1e-5), warmup=args.warmup, iters=args.iters)
        row["norm_shard"] = time_us(lambda: ops.add_rmsnorm_(scratch[:rpr], res[:rpr], w, 1e-5), warmup=args.warmup, iters=args.iters)
        if W > 1:
            row["nccl_ar"] = time_us(lambda: dist.all_reduce(view), **kw)

            def nccl_norm():
                dist.all_reduce(view)
                ops.add_rmsnorm_(view, res, w, 1e-5)
            row["nccl_ar_norm"] = time_us(nccl_norm, **kw)
            best = {}
            for name, fn in (("mm_ar", comm.all_reduce_), ("mm_rs", comm.reduce_scatter_), ("mm_ag", comm.all_gather_)):
                best[name] = min(time_us(lambda: fn(view, c), **kw) for c in args.ctas)
            row.update(best)
            row["simple_fusion"] = min(time_us(lambda: comm.fused_allreduce_add_rmsnorm_(view, res, w, 1e-5, c, mode=2), **kw)
                                       for c in args.ctas)
        fused = {}
        for c in args.ctas:
            fused[c] = time_us(lambda: comm.fused_allreduce_add_rmsnorm_(view, res, w, 1e-5, c), **kw)
            row[f"fused_{c}"] = fused[c]
        row["fused_best"] = min(fused.values())
        if args.burst > 0:
            cb = min(fused, key=fused.get)
            row["fused_burst"] = burst_us(lambda: comm.fused_allreduce_add_rmsnorm_(view, res, w, 1e-5, cb), args.burst)
            if W > 1:
                row["nccl_ar_norm_burst"] = burst_us(nccl_norm, args.burst)
        row["best_ctas"] = min(fused, key=fused.get)
        if ref_ops is not None and ok:
            # the reference kernel works on this rank's shard rows and is given the multicast address of the shard
            rview = ref_buf.tensor[:T]
            rres = res0.clone()
            off = rank * rpr * H * 2
            mc, pads = ref_buf.multicast_ptr + off, ref_buf.signal_pads_dev
            sl = slice(rank * rpr, (rank + 1) * rpr)

            def ref_refill():
                rview.copy_(x)

            def ref_fused_fn(c):
                ref_ops.fused_rs_ln_ag_cta(rview[sl], rres[sl], w, mc, pads, rank, W, c, 1e-5)
            ref_refill()
            rres.copy_(res0)
            torch.cuda.synchronize()
            dist.barrier()
            ref_fused_fn(16)
            torch.cuda.synchronize()
            rok = torch.tensor([int(torch.allclose(rview.float(), expect.float(), atol=4e-2, rtol=4e-2))], device="cuda")
            dist.all_reduce(rok, op=dist.ReduceOp.MIN)
            row["ref_correct"] = bool(rok.item())
            rkw = dict(warmup=args.warmup, iters=args.iters, before=ref_refill, sync_ranks=args.sync_ranks)
            rf = {c: time_us(lambda: ref_fused_fn(c), **rkw) for c in args.ctas}
            for c, v in rf.items():
                row[f"ref_fused_{c}"] = v
            row["ref_fused_best"] = min(rf.values())
            row["ref_mm_ar"] = min(time_us(lambda: ref_ops.multimem_ar_cta(rview[sl], mc, pads, rank, W, c), **rkw)
                                   for c in args.ctas)
            row["ref_simple_fusion"] = min(
                time_us(lambda: ref_ops.simple_fusion_rs_ln_ag_cta(rview[sl], rres[sl], w, mc, pads, rank, W, c, 1e-5), **rkw)
                for c in args.ctas)
            if args.burst > 0:
                cb = min(rf, key=rf.get)
                row["ref_fused_burst"] = burst_us(lambda: ref_fused_fn(cb), args.burst)
            row["vs_ref_fused"] = row["ref_fused_best"] / row["fused_best"]
        roof = T * H * 2 / (NVLINK_GBS_MEASURED * 1e9) * 1e6 if W > 1 else 0.0
        row["roofline_us"] = roof
        row["roofline_frac"] = (roof / row["fused_best"]) if W > 1 else None
        rows.append(row)
        if rank == 0:
            print({k: (round(v, 1) if isinstance(v, float) else v) for k, v in row.items()}, flush=True)
    ops.check_status()
    if rank == 0:
        write_rows(args.out, f"fused_microbench_w{W}", rows)
    finish_ranks()


if __name__ == "__main__":
    main()
