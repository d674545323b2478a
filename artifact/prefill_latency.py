#!/usr/bin/env python
"""Prefill latency through ``LLM.generate`` (figures 1, 2, 3 and 11 of the paper; reference:
artifact/figure_2_11/bench.py:39-124): one prompt of N random token ids, ``max_tokens=1``, mean wall-clock
of ``--iters`` calls after ``--warmup`` calls, plus the device time of the same calls (CUDA events, max
over ranks). Prints ``Input length: N, Avg latency (ms): L`` lines like the reference and writes CSV.

Launch under ``torch.distributed.run`` for TP > 1. ``--modes`` selects the schedules to compare:
overlap (TokenWeave), fuse_only, baseline_multimem, baseline_nccl, no_ar (numerically wrong upper bound)."""
from __future__ import annotations

import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import RESULTS_DIR, write_rows  # noqa: E402

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def run_mode(args, mode: str, world: int, rank: int) -> list[dict]:
    from tokenweave_b200 import LLM, SamplingParams, ops
    max_len = max(args.lengths)
    llm = LLM(args.model, tensor_parallel_size=world, skip_tokenizer_init=True, enforce_eager=True,
              distributed_executor_backend="external_launcher" if world > 1 else "uni",
              max_num_batched_tokens=max_len, max_model_len=max_len + 64, block_size=128, load_format="dummy",
              tokenweave_mode=mode, num_gpu_blocks_override=(max_len + 64) // 128 + 8,
              num_hidden_layers_override=args.layers, tokenweave_config=args.config,
              tokenweave_split_offset=args.split_offset, tokenweave_attention_ctas=args.attention_ctas,
              tokenweave_mlp_ctas=args.mlp_ctas, fuse_only_ctas=args.fuse_only_ctas)
    cfg = llm.llm_engine.config.model
    runner = llm.llm_engine.core.executor.worker.runner
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    g = torch.Generator().manual_seed(0)
    rows = []
    for n in args.lengths:
        prompt = torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
        for _ in range(args.warmup):
            llm.generate(prompt_token_ids=[prompt], sampling_params=sp)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        runner.timing_events = []
        t0 = time.perf_counter()
        for _ in range(args.iters):
            llm.generate(prompt_token_ids=[prompt], sampling_params=sp)
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) / args.iters * 1e3
        dev_ms = sum(a.elapsed_time(b) for a, b in runner.timing_events) / args.iters
        runner.timing_events = None
        t = torch.tensor([wall_ms, dev_ms], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        wall_ms, dev_ms = t.tolist()
        plan = runner.planner.plan(n)
        rows.append({"model": args.model, "tp": world, "mode": mode, "tokens": n, "latency_ms": wall_ms,
                     "device_ms": dev_ms, "overlap": plan.overlap, "split": plan.split,
                     "attention_ctas": plan.attention_ctas, "mlp_ctas": plan.mlp_ctas, "layers": cfg.num_layers})
        if rank == 0:
            print(f"[{mode}] Input length: {n}, Avg latency (ms): {wall_ms:.3f} (device {dev_ms:.3f})", flush=True)
            # rows so far, so that a run cut short still leaves its measurements behind
            write_rows(args.out, f"prefill_{args.model}_tp{world}_{mode}_partial", rows)
    ops.check_status()
    llm.shutdown()
    return rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.3-70b")
    ap.add_argument("--lengths", type=int, nargs="+", default=[1024, 2048, 4096, 8192, 16384, 32768])
    ap.add_argument("--modes", nargs="+", default=["overlap", "fuse_only", "baseline_multimem", "baseline_nccl", "no_ar"])
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--config", default=None)
    ap.add_argument("--split-offset", type=int, default=None)
    ap.add_argument("--attention-ctas", type=int, default=None)
    ap.add_argument("--mlp-ctas", type=int, default=None)
    ap.add_argument("--fuse-only-ctas", type=int, default=16)
    ap.add_argument("--out", default=os.path.join(RESULTS_DIR, "prefill_latency"))
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    rows = []
    for mode in args.modes:
        if world == 1 and mode != args.modes[0]:
            break                     # a single GPU has no collective to vary
        rows += run_mode(args, mode, world, rank)
    if rank == 0:
        write_rows(args.out, f"prefill_{args.model}_tp{world}", rows)


if __name__ == "__main__":
    main()
