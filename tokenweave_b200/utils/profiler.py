"""Layer-wise / op-wise profile (counterpart of vllm/profiler/layerwise_profile.py and
tools/profiler/print_layerwise_table.py): every kernel launcher call is bracketed with CUDA events on
its stream and the device time is summed per op; GEMMs are split by shape.

    with op_profile() as prof:
        llm.generate(...)
    print(prof.table())

Events on a stream that runs concurrently with another stream (the overlap schedule) measure that
kernel's own span, so the column can add up to more than the wall time of the step.
"""
from __future__ import annotations

import contextlib

from ..ops import _native


class OpProfile:
    def __init__(self):
        self.rows: dict = {}

    def collect(self) -> None:
        for k, (n, ms) in _native.op_timing_summary().items():
            c, t = self.rows.get(k, (0, 0.0))
            self.rows[k] = (c + n, t + ms)

    def table(self) -> str:
        total = sum(t for _, t in self.rows.values()) or 1.0
        lines = [f"{'op':44s} {'calls':>8s} {'ms':>10s} {'share':>7s} {'us/call':>9s}"]
        for k, (n, t) in sorted(self.rows.items(), key=lambda kv: -kv[1][1]):
            lines.append(f"{k:44s} {n:8d} {t:10.3f} {100 * t / total:6.1f}% {1e3 * t / max(n, 1):9.1f}")
        lines.append(f"{'total':44s} {sum(n for n, _ in self.rows.values()):8d} {total:10.3f}")
        return "\n".join(lines)


@contextlib.contextmanager
def op_profile():
    prof = OpProfile()
    _native.enable_op_timing(True)
    try:
        yield prof
    finally:
        prof.collect()
        _native.enable_op_timing(False)
