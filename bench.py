#!/usr/bin/env python
"""Headline benchmark: prefill throughput of Llama-3.3-70B (bf16, random-init weights, synthetic
random-token prompt) through the public ``LLM.generate`` API, tensor-parallel over N GPUs of one node.

One step = one ``LLM.generate`` call on one prompt of ``--prompt-len`` tokens with ``max_tokens=1``
(the reference's prefill-latency methodology, artifact/figure_2_11/bench.py:52-124). Two numbers come
out of the same K timed steps:

* ``value``     tokens/s from CUDA events around the device work of each step (embedding -> decoder
                stack -> LM head -> sampling), max over ranks;
* ``e2e.value`` tokens/s from the host clock around the ``generate`` calls, which includes the
                host->device copy of the step's token ids and attention metadata from pinned memory and
                the device->host read of the sampled token.

N > 1 is launched by ``torch.distributed.run`` (one rank per GPU, NCCL); every rank runs the same engine
on the same request stream. ``--impl reference`` runs the unmodified reference from ``baseline/_ref``
when it could be installed, else prints why it is unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Llama-3.3-70B, 8192-token prefill, TokenWeave on 8xH100: 279.8 ms (artifact/csvs/figure_11a.csv:5)
BASELINE_TOKENS_PER_S = {8192: 8192 / 0.2798, 4096: 4096 / 0.1422, 2048: 2048 / 0.0767, 1024: 1024 / 0.0462,
                         16384: 16384 / 0.5853, 32768: 32768 / 1.3260}

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3.3-70b")
    ap.add_argument("--prompt-len", type=int, default=8192)
    ap.add_argument("--mode", default="overlap",
                    choices=["overlap", "fuse_only", "fused_gemm", "baseline_nccl", "baseline_custom_ar", "baseline_multimem",
                             "no_ar"])
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (marks the result invalid)")
    ap.add_argument("--cuda-graphs", dest="cuda_graphs", action="store_true", default=None,
                    help="replay the step from a CUDA graph (captured during warm-up; the default when --warmup >= 3)")
    ap.add_argument("--no-cuda-graphs", dest="cuda_graphs", action="store_false",
                    help="launch every kernel of the timed steps eagerly")
    return ap.parse_args()


class ClockSampler:
    def __init__(self, enabled: bool):
        self.proc = None
        self.path = None
        if enabled:
            try:
                fd, self.path = tempfile.mkstemp(suffix=".csv")
                os.close(fd)
                self.proc = subprocess.Popen(
                    ["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                    stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            except Exception:
                self.proc = None

    def stop(self, gpu_indices):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9 or not f[0].isdigit() or int(f[0]) not in gpu_indices:
                    continue
                try:
                    sm, smax, power = float(f[1]), float(f[2]), float(f[3])
                except ValueError:
                    continue
                if power < 250:        # idle sample (between steps / before the first launch)
                    continue
                clocks.append(sm)
                mx = smax
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if clocks:
            out["sm_mhz"] = statistics.median(clocks)
            out["sm_max_mhz"] = mx
            out["samples"] = len(clocks)
        out["reasons"] = sorted(reasons)
        return out


def run_reference(args) -> None:
    """The unmodified reference (a vLLM fork) installed under baseline/_ref, through its own ``LLM.generate``:
    the same prompts, ``max_tokens=1``, eager mode, custom all-reduce off, dummy weights - the settings of its
    artifact/figure_2_11/bench.py:52-124 - timed with the same barrier + synchronize bracket as this build's arm.
    Prints the ``unavailable`` line when the fork is not installed (its build needs packages and git clones this
    image cannot supply; ``baseline/REFERENCE_INSTALL.txt`` has the record)."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    rank = int(os.environ.get("RANK", "0"))

    def unavailable(reason: str) -> None:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": reason}))

    if not os.path.isdir(os.path.join(ref_dir, "vllm")):
        note = os.path.join(ROOT, "baseline", "REFERENCE_INSTALL.txt")
        reason = "reference not installed under baseline/_ref"
        if os.path.exists(note):
            reason = open(note).read().strip().splitlines()[0]
        return unavailable(reason)
    if args.gpus > 1 and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # the fork spawns its own tensor-parallel workers; under a torchrun launch only rank 0 drives it
        if rank != 0:
            return
        for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_PORT", "TORCHELASTIC_RUN_ID"):
            os.environ.pop(k, None)
    try:
        sys.path.insert(0, ref_dir)
        import torch
        import vllm
        import vllm._C  # noqa: F401  (the compiled kernels the TokenWeave path needs)
        from vllm import LLM as RefLLM, SamplingParams as RefSamplingParams
    except Exception as e:
        return unavailable(f"reference under baseline/_ref does not import: {type(e).__name__}: {str(e)[:120]}")
    T = args.prompt_len
    hf_names = {"llama-3.3-70b": "meta-llama/Llama-3.3-70B-Instruct", "qwen2.5-72b": "Qwen/Qwen2.5-72B-Instruct",
                "mixtral-8x22b": "mistralai/Mixtral-8x22B-Instruct-v0.1"}
    try:
        llm = RefLLM(model=hf_names.get(args.model, args.model), tensor_parallel_size=args.gpus, load_format="dummy",
                     enforce_eager=True, disable_custom_all_reduce=True, enable_chunked_prefill=True,
                     enable_prefix_caching=False, max_num_batched_tokens=T, max_model_len=T + 64, dtype="bfloat16",
                     skip_tokenizer_init=True, seed=0)
    except Exception as e:
        return unavailable(f"reference engine did not start: {type(e).__name__}: {str(e)[:120]}")
    g = torch.Generator().manual_seed(1234)
    vocab = llm.llm_engine.model_config.get_vocab_size()
    prompts = [torch.randint(0, vocab, (T,), generator=g).tolist() for _ in range(args.steps + args.warmup)]
    sp = RefSamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, detokenize=False)
    for i in range(args.warmup):
        llm.generate(prompt_token_ids=[prompts[i]], sampling_params=sp, use_tqdm=False)
    sampler = ClockSampler(True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    wall = 0.0
    for i in range(args.steps):
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        llm.generate(prompt_token_ids=[prompts[args.warmup + i]], sampling_params=sp, use_tqdm=False)
        torch.cuda.synchronize()
        wall += time.perf_counter() - t0
    clocks = sampler.stop(set(range(args.gpus)))
    value = T * args.steps / wall
    base = BASELINE_TOKENS_PER_S.get(T) if args.model == "llama-3.3-70b" else None
    print(json.dumps({
        "metric": "prefill_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": wall * 1e3 / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": (value / base) if base else None, "dtype": "bf16",
        "data": "synthetic random token ids, random-init weights (load_format=dummy)",
        "config": {"model": args.model, "global_batch": 1, "seq_len": T, "parallelism": f"tp{args.gpus}",
                   "timing": "host clock around LLM.generate (the fork runs its workers in other processes)"},
        "clocks": clocks, "e2e": {"value": value, "unit": "tokens/s"}, "impl": "reference"}), flush=True)


def main() -> None:
    args = parse_args()
    if args.cuda_graphs is None:
        # eager on the first sight of a step shape, capture on the second, replay from the third on
        args.cuda_graphs = args.warmup >= 3
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist
    from tokenweave_b200 import LLM, SamplingParams, ops
    from tokenweave_b200.ops import _native

    n = args.gpus
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if n > 1 and world != n:
        raise SystemExit(f"--gpus {n} needs WORLD_SIZE={n} (launch with torch.distributed.run), got {world}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    T = args.prompt_len
    llm = LLM(args.model, tensor_parallel_size=n, skip_tokenizer_init=True, enforce_eager=True,
              distributed_executor_backend="external_launcher" if n > 1 else "uni",
              max_num_batched_tokens=T, max_model_len=T + 64, block_size=128, enable_chunked_prefill=True,
              enable_prefix_caching=False, load_format="dummy", tokenweave_mode=args.mode,
              num_gpu_blocks_override=(T + 64) // 128 + 8, num_hidden_layers_override=args.layers, seed=0,
              tokenweave_cuda_graphs=args.cuda_graphs)
    cfg = llm.llm_engine.config.model
    runner = llm.llm_engine.core.executor.worker.runner
    g = torch.Generator().manual_seed(1234)
    pinned_prompts = [torch.randint(0, cfg.vocab_size, (T,), generator=g, dtype=torch.int32).pin_memory()
                      for _ in range(args.steps + args.warmup)]
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm_launches = 0
    for i in range(args.warmup):
        l0 = _native.launch_count()
        llm.generate(prompt_token_ids=[pinned_prompts[i].tolist()], sampling_params=sp)
        if i == 0:
            warm_launches = _native.launch_count() - l0
    barrier()
    ops.check_status()

    sampler = ClockSampler(rank == 0)
    runner.timing_events = []
    launches0 = _native.launch_count()
    wall = 0.0
    h2d = d2h = 0
    barrier()
    for i in range(args.steps):
        flush.zero_()
        torch.cuda.synchronize()
        ids = pinned_prompts[args.warmup + i].tolist()
        t0 = time.perf_counter()
        out = llm.generate(prompt_token_ids=[ids], sampling_params=sp)
        torch.cuda.synchronize()
        wall += time.perf_counter() - t0
        assert len(out) == 1 and len(out[0].outputs[0].token_ids) == 1
        h2d += runner.h2d_bytes_last_step
        d2h += runner.d2h_bytes_last_step
    barrier()
    launches = _native.launch_count() - launches0
    if args.cuda_graphs:
        # replayed steps launch the kernels recorded at capture time: count those (the eager warm-up step's)
        launches = warm_launches * args.steps
    dev_ms = sum(a.elapsed_time(b) for a, b in runner.timing_events)
    assert len(runner.timing_events) == args.steps, "one engine step per generate call expected"
    runner.timing_events = None
    clocks = sampler.stop(set(range(n)))
    ops.check_status()

    t = torch.tensor([dev_ms, wall * 1e3], dtype=torch.float64, device="cuda")
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = t.tolist()
    tokens = T * args.steps
    value = tokens / (dev_ms / 1e3)
    e2e = tokens / (wall_ms / 1e3)
    base = BASELINE_TOKENS_PER_S.get(T) if args.model == "llama-3.3-70b" else None
    transport = "none"
    if n > 1:
        transport = "nvls-multimem" if runner.model.rt.comm.use_mc else ("peer" if runner.model.rt.comm.in_kernel else "nccl")
    line = {
        "metric": "prefill_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": (value / base) if base else None, "dtype": "bf16",
        "data": "synthetic random token ids, random-init weights (no checkpoint)",
        "config": {"model": args.model, "global_batch": 1, "seq_len": T, "parallelism": f"tp{n}",
                   "layers": cfg.num_layers, "tokenweave_mode": args.mode if n > 1 else "single-gpu",
                   "transport": transport, "cuda_graphs": bool(args.cuda_graphs),
                   "l2": "per-rank weights (>= 17 GB) exceed the 126 MB L2; a 256 MB buffer is zeroed between steps",
                   "baseline": "TokenWeave on 8xH100, same prompt length (artifact/csvs/figure_11a.csv)"},
        "clocks": clocks,
        # device time in SM cycles: compares runs whose clocks differ under the power cap (ms x median SM MHz)
        "cycles_per_step": (dev_ms / args.steps * 1e-3 * clocks["sm_mhz"] * 1e6) if clocks.get("sm_mhz") else None,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": wall_ms / args.steps,
                "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps},
        "gpu_launches": launches,
        "impl": "ours",
    }
    if args.layers:
        line["invalid"] = "reduced layer count (debug run)"
    if rank == 0:
        print(json.dumps(line), flush=True)
    llm.shutdown()


if __name__ == "__main__":
    main()
