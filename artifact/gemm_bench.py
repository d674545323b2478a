#!/usr/bin/env python
"""GEMM kernels on the linear-layer shapes of the served models against the library GEMMs of the box:
bf16 ``tw_gemm_bf16`` vs ``torch.matmul`` (cuBLAS), the SwiGLU-epilogue GEMM vs cuBLAS + a separate
activation kernel, and the e4m3 ``tw_gemm_fp8`` vs ``torch._scaled_mm`` (cuBLASLt fp8). Single GPU.
Prints one line per shape and writes ``results/gemm_bench/gemm_bench.csv`` (``TW_RESULTS_DIR`` overrides the folder). TFLOP/s fractions are
relative to the measured cuBLAS bf16 burst throughput of ``MEASURED_PEAKS.json`` when present.

    python artifact/gemm_bench.py --models llama-3.3-70b --tp 8 --tokens 4096 8192
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import RESULTS_DIR, measured_peaks, time_us, write_rows  # noqa: E402
from gemm_tune import shapes_for  # noqa: E402

import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--models", nargs="+", default=["llama-3.3-70b", "qwen2.5-72b", "mixtral-8x22b"])
    ap.add_argument("--tp", type=int, nargs="+", default=[8])
    ap.add_argument("--tokens", type=int, nargs="+", default=[1024, 4096, 8192])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--fp8", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--fp8-plans", type=int, nargs="*", default=[],
                    help="also time tw_gemm_fp8 with these plans (kernel * 1000 + tile width; 1 = single-CTA tiles, "
                         "2 = CTA pairs), one column each")
    ap.add_argument("--square", type=int, nargs="*", default=[8192], help="extra M=N=K problems")
    ap.add_argument("--out", default=os.path.join(RESULTS_DIR, "gemm_bench"))
    args = ap.parse_args()
    from tokenweave_b200 import ops
    from tokenweave_b200.config import resolve_model_config
    torch.cuda.set_device(0)
    peak = measured_peaks()
    todo = []
    for m in args.models:
        cfg = resolve_model_config(m)
        for tp in args.tp:
            if cfg.num_q_heads % tp:
                continue
            for s in shapes_for(cfg, tp):
                if s not in todo:
                    todo.append(s)
    problems = [(M, N, K, sw) for (N, K, sw) in todo for M in args.tokens] + [(s, s, s, 0) for s in args.square]
    rows = []
    for (M, N, K, sw) in problems:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(2 * N if sw else N, K, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * (2 * N if sw else N) * K
        ours = time_us(lambda: ops.gemm(a, w, out=out, swiglu=bool(sw)), warmup=3, iters=args.iters)
        wt = w.t()
        if sw:
            tmp = torch.empty(M, 2 * N, device="cuda", dtype=torch.bfloat16)

            def lib():
                torch.matmul(a, wt, out=tmp)
                ops.swiglu(tmp, out=out)
        else:
            def lib():
                torch.matmul(a, wt, out=out)
        cublas = time_us(lib, warmup=3, iters=args.iters)
        row = {"M": M, "N": N, "K": K, "swiglu": sw, "tw_bf16_us": round(ours, 1), "cublas_bf16_us": round(cublas, 1),
               "tw_bf16_tflops": round(flops / ours / 1e6, 1), "speedup_vs_cublas": round(cublas / ours, 3),
               "frac_of_peak": round(flops / ours / 1e6 / peak["bf16_tflops"], 3), "peak_source": peak["source"]}
        if args.fp8:
            aq, a_s = ops.quant_fp8(a)
            wq, w_s = ops.quant_fp8(w)
            f8 = time_us(lambda: ops.gemm_fp8(aq, wq, a_s, w_s, out=out, swiglu=bool(sw)), warmup=3, iters=args.iters)
            row.update(tw_fp8_us=round(f8, 1), tw_fp8_tflops=round(flops / f8 / 1e6, 1))
            for plan in args.fp8_plans:
                if sw and plan % 1000 > 256:
                    continue                                  # the SwiGLU epilogue has no wide tiles
                t = time_us(lambda: ops.gemm_fp8(aq, wq, a_s, w_s, out=out, swiglu=bool(sw), plan=plan), warmup=3,
                            iters=args.iters)
                row[f"tw_fp8_plan{plan}_us"] = round(t, 1)
            if not sw:
                try:
                    wqt = wq.t()
                    sa, sb = a_s.view(M, 1), w_s.view(1, N)
                    lt = time_us(lambda: torch._scaled_mm(aq, wqt, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16),
                                 warmup=3, iters=args.iters)
                    row.update(cublaslt_fp8_us=round(lt, 1))
                except Exception as e:  # library refuses the shape / scaling mode
                    row.update(cublaslt_fp8_us=f"n/a ({type(e).__name__})")
                # int8 operands, int32 accumulation: tw_gemm_int8 (scales applied in the epilogue, bf16 out) against
                # the library's plain int8 GEMM (int32 out, no scaling pass counted)
                ai, ai_s = ops.quant_int8(a)
                wi, wi_s = ops.quant_int8(w)
                i8 = time_us(lambda: ops.gemm_int8(ai, wi, ai_s, wi_s, out=out), warmup=3, iters=args.iters)
                row.update(tw_int8_us=round(i8, 1), tw_int8_tops=round(flops / i8 / 1e6, 1))
                try:
                    wit = wi.t()
                    lt8 = time_us(lambda: torch._int_mm(ai, wit), warmup=3, iters=args.iters)
                    row.update(cublaslt_int8_us=round(lt8, 1))
                except Exception as e:
                    row.update(cublaslt_int8_us=f"n/a ({type(e).__name__})")
        rows.append(row)
        print(" ".join(f"{k}={v}" for k, v in row.items() if k != "peak_source"), flush=True)
        del a, w, out
    ops.check_status()
    write_rows(args.out, "gemm_bench", rows)


if __name__ == "__main__":
    main()
