"""Tuned GEMM plans: which kernel (single-CTA tiles or CTA pairs) and which tile width to use for a
problem shape. The analogue of the reference's per-device tuned config files for its fused-MoE kernel
(vllm/model_executor/layers/fused_moe/configs/*.json, looked up by shape and device name,
fused_moe.py:625-674).

``gemm_configs/<device>.json`` holds ``{"<N>,<K>,<swiglu>": [[M, sms, kernel, bn, microseconds], ...]}``
written by ``artifact/gemm_tune.py`` (``NVIDIA_B200.json`` for bf16 operands, ``NVIDIA_B200_fp8.json`` for e4m3
operands). A lookup takes the entry with the nearest M (on a log scale)
among those measured with the nearest SM budget; shapes that were never tuned fall back to the cost
model inside the launcher (plan hint 0).
"""
from __future__ import annotations

import json
import math
import os
from functools import lru_cache
from pathlib import Path
from typing import Optional

CONFIG_DIR = Path(__file__).resolve().parent.parent / "gemm_configs"
_table: Optional[dict] = None
_disabled = os.environ.get("TW_GEMM_TABLE", "1") == "0"


def _load() -> dict:
    global _table
    if _table is None:
        _table = {}
        forced = os.environ.get("TW_GEMM_KERNEL")       # "1": single-CTA tiles only, "2": CTA pairs only
        if forced in ("1", "2"):
            from . import _native
            _native.load().tw_gemm_set_kernel_override(int(forced))
        for fp8, name in ((0, "NVIDIA_B200.json"), (1, "NVIDIA_B200_fp8.json")):
            path = CONFIG_DIR / name
            if path.exists() and not _disabled:
                with open(path) as f:
                    raw = json.load(f)
                for key, rows in raw.items():
                    n, k, sw = key.split(",")
                    _table[(int(n), int(k), int(sw), fp8)] = [tuple(r[:4]) for r in rows]
    return _table


def reload() -> None:
    global _table
    _table = None
    lookup.cache_clear()


def set_enabled(on: bool) -> None:
    """Turn the table off (every lookup answers 0 = cost model) or back on; tuning runs turn it off."""
    global _disabled
    _disabled = not on
    reload()


@lru_cache(maxsize=4096)
def lookup(M: int, N: int, K: int, swiglu: bool, max_ctas: int = 0, fp8: bool = False) -> int:
    """Plan hint for the launcher: ``kernel * 1000 + bn`` or 0 (let the cost model decide)."""
    rows = _load().get((N, K, int(bool(swiglu)), int(bool(fp8))))
    if not rows:
        return 0
    sms = max_ctas if max_ctas > 0 else 148
    best_sms = min({r[1] for r in rows}, key=lambda s: abs(s - sms))
    cand = [r for r in rows if r[1] == best_sms]
    m, _, kernel, bn = min(cand, key=lambda r: abs(math.log(r[0]) - math.log(max(M, 1))))
    if not (0.7 <= M / m <= 1.45):
        return 0                      # too far from anything measured
    return int(kernel) * 1000 + int(bn)
