#!/usr/bin/env python
"""Offline serving throughput (figures 12 and 13 of the paper; reference: artifact/figure_12/bench.py):
``--num-prompts`` requests of fixed (input, output) lengths with random token ids, chunked prefill with
token budget ``--max-num-batched-tokens``; reports requests/s, total (prompt + output) tokens/s and
output tokens/s, in the reference's ``Throughput: ...`` line format.

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
                  max_model_len=args.input_len + args.output_len + 64, block_size=128, load_format="dummy",
                  tokenweave_mode=mode, num_hidden_layers_override=args.layers, enable_prefix_caching=False,
                  tokenweave_cuda_graphs=args.cuda_graphs)
        vocab = llm.llm_engine.config.model.vocab_size
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, vocab, (args.input_len,), generator=g).tolist() for _ in range(args.num_prompts)]
        sp = SamplingParams(temperature=1.0, top_p=1.0, ignore_eos=True, max_tokens=args.output_len, seed=0)
        llm.generate(prompt_token_ids=prompts[:2], sampling_params=sp)          # warm-up
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
        n_out = sum(len(o.outputs[0].token_ids) for o in outs)
        n_in = sum(len(o.prompt_token_ids) for o in outs)
        row = {"model": args.model, "tp": world, "mode": mode, "input_len": args.input_len,
               "output_len": args.output_len, "num_prompts": len(outs), "chunk_budget": args.max_num_batched_tokens,
               "cuda_graphs": bool(args.cuda_graphs),
               "requests_per_s": len(outs) / dt, "total_tokens_per_s": (n_in + n_out) / dt,
               "output_tokens_per_s": n_out / dt, "elapsed_s": dt}
        rows.append(row)
        if rank == 0:
            print(f"[{mode}] Throughput: {row['requests_per_s']:.2f} requests/s, {row['total_tokens_per_s']:.2f} total tokens/s, "
                  f"{row['output_tokens_per_s']:.2f} output tokens/s", flush=True)
        ops.check_status()
        llm.shutdown()
    if rank == 0:
        write_rows(args.out, f"throughput_{args.model}_tp{world}_{args.input_len}_{args.output_len}", rows)


if __name__ == "__main__":
    main()
