#!/usr/bin/env python
"""Output agreement between schedules (reference: artifact/correctness_check/run.sh:18-95, which dumps
the texts of ``baseline_multimem`` and ``overlap_fused`` for eyeballing). Here the check is numeric: the
same prompts run under every schedule, chunked at ``--chunk`` tokens, and the greedy tokens and
first-token logits are compared with the first schedule's. ``no_ar`` is expected to differ (it deletes
the communication). Launch under ``torch.distributed.run`` for TP > 1."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--modes", nargs="+", default=["baseline_nccl", "baseline_multimem", "fuse_only", "overlap"])
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--num-prompts", type=int, default=8)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--layers", type=int, default=None)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    from tokenweave_b200 import LLM, SamplingParams, ops
    results = {}
    for mode in args.modes:
        llm = LLM(args.model, tensor_parallel_size=world, skip_tokenizer_init=True,
                  distributed_executor_backend="external_launcher" if world > 1 else "uni",
                  max_num_batched_tokens=args.chunk, max_model_len=8192, block_size=128, load_format="dummy",
                  tokenweave_mode=mode, num_hidden_layers_override=args.layers, seed=0)
        vocab = llm.llm_engine.config.model.vocab_size
        runner = llm.llm_engine.core.executor.worker.runner
        runner.capture_logits = True
        g = torch.Generator().manual_seed(0)
        lens = torch.randint(64, 3000, (args.num_prompts,), generator=g).tolist()
        prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0, max_tokens=args.max_tokens, ignore_eos=True))
        first = {}
        for reqs, logits in runner.captured_logits:
            for rid, row in zip(reqs, logits):
                first.setdefault(rid, row)
        results[mode] = ([o.outputs[0].token_ids for o in outs], torch.stack([first[str(i)] for i in range(len(prompts))]))
        ops.check_status()
        llm.shutdown()
    base = args.modes[0]
    ok = True
    for mode in args.modes[1:]:
        same = sum(a == b for a, b in zip(results[mode][0], results[base][0]))
        first_same = sum(a[0] == b[0] for a, b in zip(results[mode][0], results[base][0]))
        diff = (results[mode][1] - results[base][1]).abs().max().item()
        scale = results[base][1].abs().max().item()
        if rank == 0:
            print(f"{mode} vs {base}: {same}/{args.num_prompts} identical continuations, {first_same}/{args.num_prompts} "
                  f"identical first tokens, max |dlogit| {diff:.4f} (max |logit| {scale:.2f})", flush=True)
        if not mode.startswith("no_") and diff > 0.1 * max(1.0, scale):
            ok = False
    if rank == 0:
        print("CORRECTNESS", "PASS" if ok else "FAIL")
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
