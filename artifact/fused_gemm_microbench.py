#!/usr/bin/env python
"""The GEMM kernels that are fused with their collective, against the same work done by two kernels
(torchrun, no engine):

  gemm_rs_norm   o_proj / down_proj GEMM -> reduce-scatter -> residual add -> RMSNorm   (tw_gemm_rs_norm)
                 vs. tw_gemm_bf16 followed by the stand-alone fused collective without its all-gather
  ag_gemm        all-gather -> QKV / gate_up GEMM (+SwiGLU)                              (tw_ag_gemm)
                 vs. the in-kernel all-gather followed by tw_gemm_bf16

on the per-rank shapes of a model at this job's tensor-parallel size. Reports microseconds (CUDA events, cold
L2, median, max over ranks), the roofline of the fused op — the slower of its FLOPs at the measured cuBLAS
bf16 throughput and its NVLink bytes (T x H x 2 x (W-1)/W per direction per GPU) at the measured 770 GB/s —
and the achieved fraction. Checks the fused result against the two-kernel result.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 artifact/fused_gemm_microbench.py
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import (NVLINK_GBS_MEASURED, RESULTS_DIR, finish_ranks, init_ranks, measured_peaks, time_us,  # noqa: E402
                    write_rows)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.3-70b")
    ap.add_argument("--tokens", type=int, nargs="+", default=[1024, 4096, 8192])
    ap.add_argument("--comm-ctas", type=int, nargs="+", default=[8, 16])
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--out", default=os.path.join(RESULTS_DIR, "fused_gemm_microbench"))
    args = ap.parse_args()
    tp = init_ranks()
    from tokenweave_b200 import ops
    from tokenweave_b200.config import resolve_model_config
    from tokenweave_b200.parallel.comm import TPCommunicator
    from tokenweave_b200.parallel.symm_mem import create_symmetric_buffer

    cfg = resolve_model_config(args.model)
    W, rank = tp.world_size, tp.rank
    H, D = cfg.hidden_size, cfg.head_dim
    hq = cfg.num_q_heads // W
    hkv = max(1, cfg.num_kv_heads // W)
    inter = cfg.intermediate_size // W
    peak = measured_peaks()
    Tmax = max(args.tokens)
    buf = create_symmetric_buffer(Tmax, H, torch.bfloat16, tp)
    comm = TPCommunicator(buf, tp, wait_budget_ms=5000)
    if comm.in_kernel:
        comm.attach_flag_buffer(create_symmetric_buffer(1, 8192, torch.bfloat16, tp, None, False))
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    gw = torch.Generator(device="cuda").manual_seed(7)
    rnd = lambda *s, gen=g, sc=1.0: (torch.randn(*s, device="cuda", generator=gen) * sc).to(torch.bfloat16)
    norm_w = (1 + 0.1 * torch.randn(H, device="cuda", generator=gw)).to(torch.bfloat16)
    rows = []
    shapes_rs = [("o_proj", hq * D), ("down_proj", inter)] if not cfg.is_moe else [("o_proj", hq * D)]
    shapes_ag = [("qkv_proj", (hq + 2 * hkv) * D, False)] + ([] if cfg.is_moe else [("gate_up_proj", inter, True)])
    for T in args.tokens:
        if T % W:
            continue
        view = buf.tensor[:T]
        nvlink_us = T * H * 2 * (W - 1) / W / (NVLINK_GBS_MEASURED * 1e9) * 1e6
        # ---- GEMM -> reduce-scatter -> add -> RMSNorm -------------------------------------------------
        for name, K in shapes_rs:
            a = rnd(T, K)
            w = rnd(H, K, sc=K ** -0.5)
            res0 = rnd(T, H, gen=torch.Generator(device="cuda").manual_seed(5))
            res = res0.clone()

            def unfused():
                ops.gemm(a, w, out=view)
                comm.fused_allreduce_add_rmsnorm_(view, res, norm_w, 1e-5, max_ctas=16, mode=1)
            res.copy_(res0)
            unfused()
            torch.cuda.synchronize()
            rpr = T // W
            want = view[rank * rpr:(rank + 1) * rpr].clone()
            res.copy_(res0)
            dist.barrier()
            comm.gemm_rs_norm_(a, w, view, T, res, norm_w, 1e-5, comm_ctas=args.comm_ctas[0])
            torch.cuda.synchronize()
            ok = torch.allclose(view[rank * rpr:(rank + 1) * rpr].float(), want.float(), atol=4e-2, rtol=4e-2)
            t_un = time_us(unfused, warmup=args.warmup, iters=args.iters)
            best = min((time_us(lambda: comm.gemm_rs_norm_(a, w, view, T, res, norm_w, 1e-5, comm_ctas=c),
                                warmup=args.warmup, iters=args.iters), c) for c in args.comm_ctas)
            flops_us = 2.0 * T * H * K / (peak["bf16_tflops"] * 1e12) * 1e6
            roof = max(flops_us, nvlink_us)
            rows.append({"op": "gemm_rs_norm", "layer": name, "tokens": T, "N": H, "K": K, "world": W, "correct": bool(ok),
                         "unfused_us": round(t_un, 1), "fused_us": round(best[0], 1), "comm_ctas": best[1],
                         "speedup": round(t_un / best[0], 3), "roofline_us": round(roof, 1),
                         "roofline_bound": "gemm" if flops_us >= nvlink_us else "nvlink",
                         "roofline_frac": round(roof / best[0], 3), "peak_source": peak["source"]})
        # ---- all-gather -> GEMM -----------------------------------------------------------------------
        for name, N, sw in shapes_ag:
            w = rnd(2 * N if sw else N, H, sc=H ** -0.5)
            out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            x = rnd(T, H)

            def refill():
                view.copy_(x)           # every rank's shard of the rows is what it would have produced itself

            def unfused():
                comm.all_gather_(view, max_ctas=16)
                ops.gemm(view, w, out=out, swiglu=sw)
            refill()
            unfused()
            torch.cuda.synchronize()
            want = out.clone()
            refill()
            dist.barrier()
            comm.ag_gemm(view, w, out, T, swiglu=sw, comm_ctas=args.comm_ctas[0])
            torch.cuda.synchronize()
            ok = torch.allclose(out.float(), want.float(), atol=4e-2, rtol=4e-2)
            t_un = time_us(unfused, warmup=args.warmup, iters=args.iters, before=refill)
            best = min((time_us(lambda: comm.ag_gemm(view, w, out, T, swiglu=sw, comm_ctas=c), warmup=args.warmup,
                                iters=args.iters, before=refill), c) for c in args.comm_ctas)
            flops_us = 2.0 * T * (2 * N if sw else N) * H / (peak["bf16_tflops"] * 1e12) * 1e6
            roof = max(flops_us, nvlink_us)
            rows.append({"op": "ag_gemm", "layer": name, "tokens": T, "N": N, "K": H, "world": W, "correct": bool(ok),
                         "unfused_us": round(t_un, 1), "fused_us": round(best[0], 1), "comm_ctas": best[1],
                         "speedup": round(t_un / best[0], 3), "roofline_us": round(roof, 1),
                         "roofline_bound": "gemm" if flops_us >= nvlink_us else "nvlink",
                         "roofline_frac": round(roof / best[0], 3), "peak_source": peak["source"]})
        if rank == 0:
            for r in rows[-(len(shapes_rs) + len(shapes_ag)):]:
                print(r, flush=True)
    ops.check_status()
    if rank == 0:
        write_rows(args.out, f"fused_gemm_microbench_w{W}", rows)
    finish_ranks()


if __name__ == "__main__":
    main()
