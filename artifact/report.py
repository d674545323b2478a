#!/usr/bin/env python
"""Turns the CSV files the benchmarks write into the tables of the paper's figures (the reference draws them with
its ``artifact/figure_*/plot.py`` scripts; this prints Markdown, which needs no plotting library):

* fused microbenchmark (figures 4 and 10): fused kernel per CTA budget, NCCL all-reduce + norm, the in-kernel
  all-reduce, the reference's own kernel where it was timed, and the speed-ups between them;
* prefill latency (figures 2 and 11): one row per prompt length, one column per schedule, speed-up of the first
  schedule over the others;
* throughput (figures 12 and 13): one row per run with the ratio to the run's baseline schedule.

    python artifact/report.py artifact/csvs            # every CSV family found under the directory
"""
from __future__ import annotations

import csv
import glob
import os
import sys
from collections import defaultdict


def _rows(path: str) -> list[dict]:
    with open(path, newline="") as f:
        return list(csv.DictReader(f))


def _f(v, digits: int = 1) -> str:
    try:
        return f"{float(v):.{digits}f}"
    except (TypeError, ValueError):
        return "—"


def _table(header: list[str], body: list[list[str]]) -> str:
    out = ["| " + " | ".join(header) + " |", "|" + "---|" * len(header)]
    out += ["| " + " | ".join(r) + " |" for r in body]
    return "\n".join(out)


def fused_table(rows: list[dict]) -> str:
    """Fused collective microbenchmark, one row per token count (microseconds)."""
    ctas = sorted((int(k.split("_")[1]) for k in rows[0] if k.startswith("fused_") and k.split("_")[1].isdigit()))
    has_ref = "ref_fused_best" in rows[0] and any(r.get("ref_fused_best") for r in rows)
    header = ["tokens", "NCCL AR + norm", "in-kernel AR"] + [f"fused, {c} CTAs" for c in ctas] + ["fused best",
                                                                                                    "vs NCCL + norm"]
    if has_ref:
        header += ["reference kernel best", "vs reference"]
    body = []
    for r in rows:
        best = float(r["fused_best"])
        line = [r["tokens"], _f(r["nccl_ar_norm"]), _f(r["mm_ar"])] + [_f(r.get(f"fused_{c}")) for c in ctas]
        line += [_f(best), _f(float(r["nccl_ar_norm"]) / best, 2) + "x"]
        if has_ref:
            ref = r.get("ref_fused_best")
            line += [_f(ref), (_f(float(ref) / best, 2) + "x") if ref else "—"]
        body.append(line)
    return _table(header, body)


def prefill_table(rows: list[dict]) -> str:
    """Prefill latency (device milliseconds), one row per prompt length, one column per schedule."""
    modes, by_len = [], defaultdict(dict)
    for r in rows:
        if r["mode"] not in modes:
            modes.append(r["mode"])
        by_len[int(r["tokens"])][r["mode"]] = float(r.get("device_ms") or r["latency_ms"])
    header = ["tokens"] + modes + [f"{modes[0]} vs {m}" for m in modes[1:]]
    body = []
    for n in sorted(by_len):
        d = by_len[n]
        line = [str(n)] + [_f(d.get(m)) for m in modes]
        line += [(_f(d[m] / d[modes[0]], 2) + "x") if m in d and modes[0] in d else "—" for m in modes[1:]]
        body.append(line)
    return _table(header, body)


def throughput_table(rows: list[dict]) -> str:
    """Offline throughput, one row per run; the ratio is against the run group's last schedule that is a baseline."""
    groups = defaultdict(list)
    for r in rows:
        groups[(r.get("model"), r.get("input_len"), r.get("output_len"), r.get("chunk_budget"), r.get("workload", ""),
                r.get("cuda_graphs", ""), r.get("engine_core_process", ""))].append(r)
    header = ["model", "input / output", "chunk budget", "schedule", "requests/s", "total tokens/s", "output tokens/s",
              "vs baseline"]
    body = []
    for key, rs in groups.items():
        base = next((float(r["total_tokens_per_s"]) for r in rs if r["mode"].startswith("baseline")), None)
        for r in rs:
            ratio = (_f(float(r["total_tokens_per_s"]) / base, 2) + "x") if base else "—"
            body.append([str(key[0]), f"{key[1]} / {key[2]}", str(key[3]), r["mode"], _f(r["requests_per_s"], 2),
                         _f(r["total_tokens_per_s"], 0), _f(r["output_tokens_per_s"], 0), ratio])
    return _table(header, body)


FAMILIES = (("fused_microbench", fused_table, "Fused reduce-scatter + add + RMSNorm + all-gather (µs)"),
            ("prefill_", prefill_table, "Prefill latency (device ms)"),
            ("throughput_", throughput_table, "Offline throughput"))


def report(directory: str) -> str:
    out = []
    for path in sorted(glob.glob(os.path.join(directory, "**", "*.csv"), recursive=True)):
        name = os.path.basename(path)
        for prefix, fn, title in FAMILIES:
            if name.startswith(prefix) and "partial" not in name:
                rows = _rows(path)
                if rows:
                    try:
                        out.append(f"### {title}: `{name}`\n\n{fn(rows)}\n")
                    except (KeyError, ValueError) as e:
                        out.append(f"### {title}: `{name}`\n\n(not in the expected layout: {e})\n")
                break
    return "\n".join(out)


if __name__ == "__main__":
    print(report(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "csvs")))
