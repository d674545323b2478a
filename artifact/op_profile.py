#!/usr/bin/env python
"""Per-op device-time breakdown of prefill steps (the layer-wise profile table). Launch under
``torch.distributed.run`` for TP > 1; rank 0 prints the table and writes it to ``--out``.

``--tp-shard N`` (single GPU): the model is cut down to what ONE rank of an N-way tensor-parallel group computes
(heads, KV heads, MLP columns and vocabulary divided by N) and runs without collectives: the compute-stream
profile of that rank, measurable where N GPUs are not at hand."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from common import RESULTS_DIR, ROOT  # noqa: E402,F401

import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.3-70b")
    ap.add_argument("--prompt-len", type=int, default=8192)
    ap.add_argument("--mode", default="overlap")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--tp-shard", type=int, default=1, help="single GPU: one rank's share of an N-way TP group")
    ap.add_argument("--out", default=os.path.join(RESULTS_DIR, "op_profile.txt"))
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    from tokenweave_b200 import LLM, SamplingParams
    from tokenweave_b200.utils.profiler import op_profile
    T = args.prompt_len
    model = args.model
    if args.tp_shard > 1:
        import dataclasses
        from tokenweave_b200.config import resolve_model_config
        full, n = resolve_model_config(args.model), args.tp_shard
        assert world == 1 and full.num_q_heads % n == 0 and full.intermediate_size % n == 0
        model = dataclasses.replace(full, name=f"{full.name}-shard{n}", num_q_heads=full.num_q_heads // n,
                                    num_kv_heads=max(1, full.num_kv_heads // n),
                                    intermediate_size=full.intermediate_size // n,
                                    vocab_size=-(-full.vocab_size // n))
    llm = LLM(model, tensor_parallel_size=world, skip_tokenizer_init=True,
              distributed_executor_backend="external_launcher" if world > 1 else "uni", max_num_batched_tokens=T,
              max_model_len=T + 64, block_size=128, load_format="dummy", tokenweave_mode=args.mode,
              num_gpu_blocks_override=(T + 64) // 128 + 8, num_hidden_layers_override=args.layers)
    vocab = llm.llm_engine.config.model.vocab_size
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    prompt = torch.randint(0, vocab, (T,), generator=torch.Generator().manual_seed(0)).tolist()
    for _ in range(2):
        llm.generate(prompt_token_ids=[prompt], sampling_params=sp)
    runner = llm.llm_engine.core.executor.worker.runner
    runner.timing_events = []
    with op_profile() as prof:
        for _ in range(args.steps):
            llm.generate(prompt_token_ids=[prompt], sampling_params=sp)
    step_ms = sum(a.elapsed_time(b) for a, b in runner.timing_events) / args.steps
    if rank == 0:
        text = (f"model {args.model}{f' (one rank of tp{args.tp_shard})' if args.tp_shard > 1 else ''} tp{world} mode {args.mode} prompt {T}: {step_ms:.2f} ms per step (device), "
                f"{args.steps} steps\n" + prof.table())
        print(text, flush=True)
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            f.write(text + "\n")
    llm.shutdown()


if __name__ == "__main__":
    main()
