#!/usr/bin/env python
"""Offline inference with TokenWeave overlap, the counterpart of the reference's
``tokenweave_offline_example.py``: long prompts (repeated text, a few thousand tokens each), tensor
parallel over the GPUs of one node, chunked prefill with a 2048-token budget.

Single GPU:   python examples/offline_inference.py --model llama-3.1-8b
Eight GPUs:   python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
                  examples/offline_inference.py --model llama-3.3-70b
              (or, from one process: --executor mp --tensor-parallel-size 8)

Without a checkpoint directory the weights are random (``load_format="dummy"``), so the text is
noise; pass a HuggingFace checkpoint directory as --model to get real completions."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tokenweave_b200 import LLM, SamplingParams  # noqa: E402

PASSAGE = ("The quick brown fox jumps over the lazy dog while the communication kernels of one half of the "
           "batch hide behind the matrix multiplications of the other half. ")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--tensor-parallel-size", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--executor", default="auto", choices=["auto", "uni", "mp", "external_launcher"])
    ap.add_argument("--mode", default="overlap")
    ap.add_argument("--max-tokens", type=int, default=32)
    ap.add_argument("--num-prompts", type=int, default=4)
    ap.add_argument("--repeat", type=int, default=40, help="copies of the passage per prompt")
    args = ap.parse_args()

    llm = LLM(model=args.model, tokenizer=None if os.path.isdir(args.model) else "byte",
              tensor_parallel_size=args.tensor_parallel_size, distributed_executor_backend=args.executor,
              enforce_eager=True, disable_custom_all_reduce=True, enable_chunked_prefill=True,
              enable_prefix_caching=False, max_num_batched_tokens=2048, max_model_len=16384,
              tokenweave_mode=args.mode)
    prompts = [f"[{i}] " + PASSAGE * args.repeat + "Continue the story:" for i in range(args.num_prompts)]
    outputs = llm.generate(prompts, SamplingParams(temperature=0.8, top_p=0.95, max_tokens=args.max_tokens, seed=0))
    if int(os.environ.get("RANK", "0")) == 0:
        for out in outputs:
            print(f"prompt ({len(out.prompt_token_ids)} tokens): {out.prompt[:60]!r}...")
            print(f"  -> {out.outputs[0].text!r}  [{out.outputs[0].finish_reason}]")
    llm.shutdown()


if __name__ == "__main__":
    main()
