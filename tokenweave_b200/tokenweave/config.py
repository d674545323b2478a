"""Per-model TokenWeave configuration files and the split planner.

File schema (same as vllm/tokenweave_configs/*.json of the reference):
``{"<tokens>": {"attention_ctas": n, "mlp_ctas": n, "split_offset": n [, "baseline_ctas": n] [, "overlap": 0|1]}}``,
(``"overlap": 0``, written by the config generator where the unsplit fused schedule measured faster, sends
token counts nearest to that key down the fuse-only path even above the model's threshold), file names ``{llama,qwen2,mixtral}_config_{tp}.json``. The entry with the key nearest to the step's
token count is used (vllm/model_executor/models/llama.py:516-520); the cut is
``round_up(T, 256) // 2 + split_offset`` (llama.py:521). The planner is the single source of truth for
the cut: the model runner builds the per-split attention metadata from the same ``SplitPlan`` the
model executes (the reference computes the formula twice, gpu_model_runner.py:622-628).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from functools import lru_cache
from pathlib import Path
from typing import Optional

from .. import envs

CONFIG_DIR = Path(__file__).resolve().parent.parent / "tokenweave_configs"
PAD_GRANULARITY = 256
DEFAULT_THRESHOLD = {"llama": 1024, "qwen2": 1024, "mixtral": 2048}
# architectures without a tuned table of their own use the table of the family with the same layer shape
CONFIG_FAMILY = {"qwen3": "qwen2", "mistral": "llama", "phi3": "llama"}


@lru_cache(maxsize=32)
def load_config(path: str) -> dict[int, dict[str, int]]:
    with open(path) as f:
        raw = json.load(f)
    return {int(k): {kk: int(vv) for kk, vv in v.items()} for k, v in raw.items()}


def default_config_path(architecture: str, tp_size: int) -> Optional[str]:
    """``<arch>_config_<tp>.json``; falls back to the nearest larger TP size that has a file."""
    for arch in (architecture, CONFIG_FAMILY.get(architecture)):
        if arch is None:
            continue
        for tp in sorted({tp_size, 8, 4, 2}, key=lambda t: (t < tp_size, abs(t - tp_size))):
            p = CONFIG_DIR / f"{arch}_config_{tp}.json"
            if p.exists():
                return str(p)
    return None


@dataclass(frozen=True)
class SplitPlan:
    num_tokens: int
    padded_tokens: int
    overlap: bool
    split: int = 0               # rows [0, split) are subset 0, [split, padded) subset 1
    attention_ctas: int = 16
    mlp_ctas: int = 16
    tail_ctas: int = 16          # last fused call of the overlap schedule (runs alone)

    @property
    def tokens_0(self) -> int:
        return min(self.split, self.num_tokens) if self.overlap else self.num_tokens

    @property
    def tokens_1(self) -> int:
        return max(0, self.num_tokens - self.split) if self.overlap else 0


class TokenWeavePlanner:
    def __init__(self, architecture: str, tp_size: int, mode: str = "overlap", config_path: Optional[str] = None,
                 threshold: Optional[int] = None, fuse_only_ctas: int = 16, split_offset: Optional[int] = None,
                 attention_ctas: Optional[int] = None, mlp_ctas: Optional[int] = None, force_overlap: bool = False):
        self.architecture = architecture
        self.tp_size = tp_size
        self.mode = mode
        self.threshold = threshold if threshold is not None else DEFAULT_THRESHOLD.get(architecture, 1024)
        self.fuse_only_ctas = fuse_only_ctas
        self.force_overlap = force_overlap
        self._override = (split_offset, attention_ctas, mlp_ctas)
        path = config_path or default_config_path(architecture, tp_size)
        self.table = load_config(path) if path else {}
        self.config_path = path

    def entry(self, num_tokens: int) -> dict[str, int]:
        base = {"attention_ctas": 8, "mlp_ctas": 8, "split_offset": 0}
        if self.table:
            key = min(self.table, key=lambda k: abs(k - num_tokens))
            base.update(self.table[key])
        off, a, m = self._override
        env_off, env_a, env_m = envs.TW_SPLIT_OFFSET, envs.TW_MAX_CTAS_ATTN, envs.TW_MAX_CTAS_MLP
        for name, cfg_v, env_v in (("split_offset", off, env_off), ("attention_ctas", a, env_a), ("mlp_ctas", m, env_m)):
            if cfg_v is not None:
                base[name] = cfg_v
            elif env_v is not None:
                base[name] = env_v
        return base

    def plan(self, num_tokens: int) -> SplitPlan:
        w = max(1, self.tp_size)
        can_overlap = self.mode == "overlap" and (self.tp_size > 1 or self.force_overlap)
        if can_overlap and num_tokens >= self.threshold:
            e = self.entry(num_tokens)
            padded = (num_tokens + PAD_GRANULARITY - 1) // PAD_GRANULARITY * PAD_GRANULARITY
            if e.get("overlap", 1) == 0 and not self.force_overlap:
                padded = 0          # tuned: the unsplit schedule is faster at this size
            split = padded // 2 + e["split_offset"]
            split = max(w, min(split, padded - w))
            split -= split % w
            if padded and 0 < split < num_tokens and (padded - split) % w == 0:
                return SplitPlan(num_tokens, padded, True, split, e["attention_ctas"], e["mlp_ctas"],
                                 16 if num_tokens < 16384 else 32)
        padded = (num_tokens + w - 1) // w * w
        ctas = self.fuse_only_ctas
        if self.table:
            key = min(self.table, key=lambda k: abs(k - num_tokens))
            ctas = self.table[key].get("baseline_ctas", ctas)
        return SplitPlan(num_tokens, padded, False, 0, ctas, ctas, ctas)
