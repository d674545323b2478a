#!/usr/bin/env python
"""TokenWeave config generator (autotuner). Reference: artifact/configs_generator/run.sh:11-137 and
generator.py:46-94, which sweep ``split_offset in {0,128,256} x attention_ctas in {2,4,8} x mlp_ctas in
{2,4,8}`` (overlap) and ``ctas in {16,32}`` (fuse-only) through full prefill-latency runs and keep the
argmin per prompt length.

This generator sweeps the same grid inside ONE engine instance per TP size: the split offset and SM
budgets are properties of the per-step plan, so each combination is a planner override, not a new
process with patched model files. Writes ``<arch>_config_<tp>.json`` in the reference's schema (plus
``baseline_ctas``) and a CSV of every measurement. Launch under ``torch.distributed.run``."""
from __future__ import annotations

import argparse
import itertools
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import RESULTS_DIR, write_rows  # noqa: E402

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.3-70b")
    ap.add_argument("--lengths", type=int, nargs="+", default=[1024, 2048, 4096, 8192, 16384, 32768])
    ap.add_argument("--split-offsets", type=int, nargs="+", default=[0, 128, 256])
    ap.add_argument("--attention-ctas", type=int, nargs="+", default=[2, 4, 8, 16])
    ap.add_argument("--mlp-ctas", type=int, nargs="+", default=[2, 4, 8, 16])
    ap.add_argument("--baseline-ctas", type=int, nargs="+", default=[16, 32])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--layers", type=int, default=None, help="tune on a truncated stack (per-layer behaviour is identical)")
    ap.add_argument("--search", default="grid", choices=["grid", "coordinate"],
                    help="grid: every combination, as the reference does; coordinate: one axis at a time from "
                         "(offset 0, 8, 8) - attention CTAs, then MLP CTAs, then the split offset (11 instead of 48 "
                         "measurements per length)")
    ap.add_argument("--out-dir", default=os.path.join(RESULTS_DIR, "configs"))
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    from tokenweave_b200 import LLM, SamplingParams, ops
    from tokenweave_b200.tokenweave.config import TokenWeavePlanner
    max_len = max(args.lengths)
    llm = LLM(args.model, tensor_parallel_size=world, skip_tokenizer_init=True,
              distributed_executor_backend="external_launcher" if world > 1 else "uni",
              max_num_batched_tokens=max_len, max_model_len=max_len + 64, block_size=128, load_format="dummy",
              tokenweave_mode="overlap", num_gpu_blocks_override=(max_len + 64) // 128 + 8,
              num_hidden_layers_override=args.layers)
    cfg = llm.llm_engine.config.model
    runner = llm.llm_engine.core.executor.worker.runner
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    g = torch.Generator().manual_seed(0)

    def measure(prompt) -> float:
        for _ in range(args.warmup):
            llm.generate(prompt_token_ids=[prompt], sampling_params=sp)
        runner.timing_events = []
        for _ in range(args.iters):
            llm.generate(prompt_token_ids=[prompt], sampling_params=sp)
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in runner.timing_events) / args.iters
        runner.timing_events = None
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def planner(mode, **kw):
        return TokenWeavePlanner(cfg.architecture, world, mode, config_path=None, threshold=0 if mode == "overlap" else None, **kw)

    rows, table = [], {}
    for n in args.lengths:
        prompt = torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
        best = None
        seen = {}

        def try_overlap(off, a, m):
            nonlocal best
            if (off, a, m) in seen:
                return seen[(off, a, m)]
            runner.planner = planner("overlap", split_offset=off, attention_ctas=a, mlp_ctas=m)
            ms = measure(prompt)
            seen[(off, a, m)] = ms
            rows.append({"tokens": n, "kind": "overlap", "split_offset": off, "attention_ctas": a, "mlp_ctas": m, "ms": ms})
            if best is None or ms < best[0]:
                best = (ms, off, a, m)
            return ms

        if args.search == "grid":
            for off, a, m in itertools.product(args.split_offsets, args.attention_ctas, args.mlp_ctas):
                try_overlap(off, a, m)
        else:
            mid = lambda xs: xs[len(xs) // 2]           # noqa: E731
            off, a, m = args.split_offsets[0], mid(args.attention_ctas), mid(args.mlp_ctas)
            a = min(args.attention_ctas, key=lambda v: try_overlap(off, v, m))
            m = min(args.mlp_ctas, key=lambda v: try_overlap(off, a, v))
            off = min(args.split_offsets, key=lambda v: try_overlap(v, a, m))
        best_base = None
        for c in args.baseline_ctas:
            runner.planner = planner("fuse_only", fuse_only_ctas=c)
            runner.planner.table = {}
            ms = measure(prompt)
            rows.append({"tokens": n, "kind": "fuse_only", "split_offset": 0, "attention_ctas": c, "mlp_ctas": c, "ms": ms})
            if best_base is None or ms < best_base[0]:
                best_base = (ms, c)
        table[str(n)] = {"attention_ctas": best[2], "mlp_ctas": best[3], "split_offset": best[1],
                         "baseline_ctas": best_base[1]}
        if best_base[0] < best[0]:
            table[str(n)]["overlap"] = 0        # the unsplit fused schedule wins at this size
        if rank == 0:
            print(f"tokens {n}: overlap best {best[0]:.2f} ms (offset {best[1]}, attn {best[2]}, mlp {best[3]}); "
                  f"fuse-only best {best_base[0]:.2f} ms ({best_base[1]} CTAs)", flush=True)
    ops.check_status()
    if rank == 0:
        os.makedirs(args.out_dir, exist_ok=True)
        with open(os.path.join(args.out_dir, f"{cfg.architecture}_config_{world}.json"), "w") as f:
            json.dump(table, f, indent=2)
        write_rows(args.out_dir, f"sweep_{cfg.architecture}_tp{world}", rows)
    llm.shutdown()


if __name__ == "__main__":
    main()
