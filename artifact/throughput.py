#!/usr/bin/env python
"""Offline serving throughput (figures 12 and 13 of the paper; reference: artifact/figure_12/bench.py):
``--num-prompts`` requests of fixed (input, output) lengths with random token ids, chunked prefill with
token budget ``--max-num-batched-tokens``; reports requests/s, total (prompt + output) tokens/s and
output tokens/s, in the reference's ``Throughput: ...`` line format. ``--workload mixed`` draws the lengths
of every request from a long-tailed distribution instead (prompts 16..2048 tokens with median near 200,
outputs 8..512 with median near 120): a synthetic stand-in for the ShareGPT conversations of the reference's
figure 12 (artifact/figure_12/bench.py:195-196), which this machine cannot download. Each row also carries
the device time of the run's engine steps, so the host share (scheduling, input preparation, sampling set-up,
detokenisation) is visible next to the throughput; ``--engine-core-process`` moves scheduler and executor
into a process of their own.

Launch under ``torch.distributed.run`` for TP > 1."""
from __future__ import annotations

import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import RESULTS_DIR, write_rows  # noqa: E402

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.3-70b")
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=128)
    ap.add_argument("--num-prompts", type=int, default=1000)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--modes", nargs="+", default=["overlap", "baseline_multimem", "no_ar"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--cuda-graphs", action="store_true", help="replay repeated step shapes (decode) from CUDA graphs")
    ap.add_argument("--workload", default="fixed", choices=["fixed", "mixed"],
                    help="fixed: every request has --input-len / --output-len; mixed: long-tailed lengths per request")
    ap.add_argument("--engine-core-process", action="store_true",
                    help="scheduler + executor in their own process (single GPU or the multiprocess executor only)")
    ap.add_argument("--out", default=os.path.join(RESULTS_DIR, "throughput"))
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    from tokenweave_b200 import LLM, SamplingParams, ops
    rows = []
    for mode in args.modes:
        llm = LLM(args.model, tensor_parallel_size=world, skip_tokenizer_init=True, enforce_eager=True,
                  distributed_executor_backend="external_launcher" if world > 1 else "uni",
                  max_num_batched_tokens=args.max_num_batched_tokens, max_num_seqs=args.max_num_seqs,
                  max_model_len=max(args.input_len + args.output_len, 2048 + 512 if args.workload == "mixed" else 0) + 64,
                  block_size=128, load_format="dummy",
                  tokenweave_mode=mode, num_hidden_layers_override=args.layers, enable_prefix_caching=False,
                  tokenweave_cuda_graphs=args.cuda_graphs, engine_core_process=args.engine_core_process)
        vocab = llm.llm_engine.config.model.vocab_size
        g = torch.Generator().manual_seed(0)
        if args.workload == "mixed":
            # log-normal lengths, clipped: most conversations are short, a few are long
            in_lens = torch.exp(torch.randn(args.num_prompts, generator=g) * 1.0 + 5.3).clamp(16, 2048).long().tolist()
            out_lens = torch.exp(torch.randn(args.num_prompts, generator=g) * 0.9 + 4.8).clamp(8, 512).long().tolist()
        else:
            in_lens, out_lens = [args.input_len] * args.num_prompts, [args.output_len] * args.num_prompts
        prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in in_lens]
        sp = [SamplingParams(temperature=1.0, top_p=1.0, ignore_eos=True, max_tokens=n, seed=0) for n in out_lens]
        llm.generate(prompt_token_ids=prompts[:2], sampling_params=sp[:2])          # warm-up
        runner = None if args.engine_core_process else llm.llm_engine.core.executor.worker.runner
        if runner is not None:
            runner.timing_events = []
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=sp)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        t = torch.tensor([dt], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
        dev_s = None
        if runner is not None:
            dev_s = sum(a.elapsed_time(b) for a, b in runner.timing_events) / 1e3
            steps = len(runner.timing_events)
            runner.timing_events = None
        n_out = sum(len(o.outputs[0].token_ids) for o in outs)
        n_in = sum(len(o.prompt_token_ids) for o in outs)
        row = {"model": args.model, "tp": world, "mode": mode, "input_len": args.input_len,
               "output_len": args.output_len, "num_prompts": len(outs), "chunk_budget": args.max_num_batched_tokens,
               "cuda_graphs": bool(args.cuda_graphs), "workload": args.workload,
               "engine_core_process": bool(args.engine_core_process),
               "device_s": dev_s, "host_share": (1.0 - dev_s / dt) if dev_s else None,
               "engine_steps": steps if dev_s else None,
               "requests_per_s": len(outs) / dt, "total_tokens_per_s": (n_in + n_out) / dt,
               "output_tokens_per_s": n_out / dt, "elapsed_s": dt}
        rows.append(row)
        if rank == 0:
            print(f"[{mode}] Throughput: {row['requests_per_s']:.2f} requests/s, {row['total_tokens_per_s']:.2f} total tokens/s, "
                  f"{row['output_tokens_per_s']:.2f} output tokens/s"
                  + (f" (device {dev_s:.2f} s of {dt:.2f} s: host share {row['host_share']:.1%})" if dev_s else ""), flush=True)
        ops.check_status()
        llm.shutdown()
    if rank == 0:
        tag = "mixed" if args.workload == "mixed" else f"{args.input_len}_{args.output_len}"
        write_rows(args.out, f"throughput_{args.model}_tp{world}_{tag}_b{args.max_num_batched_tokens}", rows)


if __name__ == "__main__":
    main()
