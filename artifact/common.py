"""Shared measurement helpers of the artifact benchmarks.

Methodology (mirrors artifact/figure_4_10/bench.py:15-61 of the reference): CUDA events around each
call on the launching stream, warm-up iterations first, a 256 MB buffer zeroed between iterations so
every timed call starts with a cold L2, the median over the timed iterations, and for multi-GPU runs
the maximum over ranks of that median (the reference reports rank 0 only).
"""
from __future__ import annotations

import csv
import json
import os
import statistics
import sys
from typing import Callable, Optional

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

RESULTS_DIR = os.environ.get("TW_RESULTS_DIR", "results")     # where the benchmarks write their CSV / JSON / logs
NVLINK_GBS_MEASURED = 770.0      # peer copy, per direction per GPU, measured on this pool
_flush = None


def l2_flush() -> None:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_us(fn: Callable[[], None], warmup: int = 10, iters: int = 100, before: Optional[Callable[[], None]] = None,
            sync_ranks: bool = False) -> float:
    """Median device time of ``fn`` in microseconds (max over ranks when a process group exists)."""
    for _ in range(warmup):
        if before:
            before()
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if before:
            before()
        l2_flush()
        if sync_ranks and dist.is_initialized():
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) * 1e3)
    med = statistics.median(times)
    if dist.is_initialized():
        t = torch.tensor([med], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        med = float(t.item())
    return med


def measured_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def init_ranks():
    """Join the torchrun job (or run single-GPU); returns the TP state."""
    from tokenweave_b200.parallel import state as pstate
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29611")
    if world > 1:
        return pstate.init_distributed(rank, world, local, "cuda")
    torch.cuda.set_device(0)
    return pstate.set_single_process(torch.device("cuda", 0))


def finish_ranks() -> None:
    from tokenweave_b200.parallel import state as pstate
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    pstate.destroy_distributed()


def write_rows(out_dir: str, name: str, rows: list[dict]) -> None:
    os.makedirs(out_dir, exist_ok=True)
    if not rows:
        return
    keys = []
    for r in rows:
        keys += [k for k in r if k not in keys]
    with open(os.path.join(out_dir, name + ".csv"), "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=keys, restval="")
        w.writeheader()
        w.writerows(rows)
    with open(os.path.join(out_dir, name + ".json"), "w") as f:
        json.dump(rows, f, indent=1)
