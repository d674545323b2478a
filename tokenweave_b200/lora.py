"""LoRA adapters at serving time: several adapters resident per worker, any mix of them (and of requests
without an adapter) in one batch.

Counterpart of vllm/lora/ (``LoRARequest``, the worker-side LoRA manager, the punica SGMV/BGMV ops): for the
rows of a batch that use adapter ``a`` a linear layer adds ``scaling * (x A_a^T) B_a^T`` to its base output.
Here that is two small tcgen05 GEMMs per adapter present in the step on gathered rows (the CPU path runs the
same code in PyTorch), applied by the decoder blocks right after the base GEMM:

* column-parallel layers (``qkv_proj``, ``gate_up_proj``): ``A`` is replicated, ``B`` keeps this rank's output
  rows; the packed projections stack their ``A`` matrices and use a block-diagonal ``B``;
* row-parallel layers (``o_proj``, ``down_proj``): ``A`` keeps this rank's input columns, ``B`` is replicated;
  the ranks' partial deltas sum up in the reduction that follows, like the base partial sums do.

Adapters are read from PEFT directories (``adapter_config.json`` + ``adapter_model.safetensors``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import ops
from .parallel.state import get_tp

_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


@dataclass(frozen=True)
class LoRARequest:
    """Names an adapter for a request (``vllm/lora/request.py``): a user-facing name, a positive integer id
    that is unique per adapter, and the PEFT directory."""
    lora_name: str
    lora_int_id: int
    lora_path: str

    def __post_init__(self):
        if self.lora_int_id < 1:
            raise ValueError("lora_int_id must be positive")


def _pad_rank(t: torch.Tensor, dim: int, mult: int = 64) -> torch.Tensor:
    """The rank dimension is the K of the second GEMM and the N of the first: pad it with zeros to one
    64-element k-block of the tcgen05 GEMM."""
    r = t.shape[dim]
    pad = (-r) % mult
    if pad == 0:
        return t.contiguous()
    shape = list(t.shape)
    shape[dim] = pad
    return torch.cat([t, torch.zeros(shape, dtype=t.dtype, device=t.device)], dim=dim).contiguous()


class LoRALayerWeights:
    """``A`` [r_total, in_local] and ``B`` [out_local, r_total] of one (possibly packed) linear layer."""

    def __init__(self, A: torch.Tensor, B: torch.Tensor):
        self.A, self.B = A, B


class LoRAAdapter:
    def __init__(self, name: str, rank: int, scaling: float, layers: dict):
        self.name, self.rank, self.scaling = name, rank, scaling
        self.layers = layers            # (layer index, "qkv_proj" | "o_proj" | "gate_up_proj" | "down_proj") -> LoRALayerWeights

    @staticmethod
    def load(path: str, model, name: str = "") -> "LoRAAdapter":
        from safetensors.torch import load_file
        with open(os.path.join(path, "adapter_config.json")) as f:
            cfg = json.load(f)
        r = int(cfg["r"])
        scaling = float(cfg.get("lora_alpha", r)) / r
        raw = load_file(os.path.join(path, "adapter_model.safetensors"))
        by_layer: dict = {}
        for key, t in raw.items():
            parts = key.split(".")
            if "layers" not in parts:
                continue
            li = int(parts[parts.index("layers") + 1])
            target = next((p for p in parts if p in _TARGETS), None)
            which = "A" if "lora_A" in parts else "B" if "lora_B" in parts else None
            if target is None or which is None:
                continue
            by_layer.setdefault(li, {}).setdefault(target, {})[which] = t
        return LoRAAdapter.from_tensors(by_layer, r, scaling, model, name or os.path.basename(path.rstrip("/")))

    @staticmethod
    def from_tensors(by_layer: dict, r: int, scaling: float, model, name: str) -> "LoRAAdapter":
        """``by_layer[layer][target] = {"A": [r, in], "B": [out, r]}`` in the unsharded HuggingFace shapes."""
        tp = get_tp()
        W, rank = max(1, tp.world_size), tp.rank
        dev = model.norm_w.device
        dt = model.cfg.dtype
        layers = {}
        for li, targets in by_layer.items():
            layer = model.layers[li]
            D = layer.attn.head_dim
            qkv = layer.qkv_proj

            def col(t):
                return t.to(device=dev, dtype=dt)
            # ---- packed q | k | v (column-parallel) ----
            present = [t for t in ("q_proj", "k_proj", "v_proj") if t in targets]
            if present:
                sizes = {"q_proj": qkv.q_heads * D, "k_proj": qkv.kv_heads * D, "v_proj": qkv.kv_heads * D}
                starts = {"q_proj": rank * qkv.q_heads * D, "k_proj": (rank // qkv.kv_replicas) * qkv.kv_heads * D,
                          "v_proj": (rank // qkv.kv_replicas) * qkv.kv_heads * D}
                offs = {"q_proj": 0, "k_proj": sizes["q_proj"], "v_proj": sizes["q_proj"] + sizes["k_proj"]}
                A = torch.cat([col(targets[t]["A"]) for t in present], dim=0)                     # [len * r, H]
                B = torch.zeros(qkv.out_per_rank, len(present) * r, dtype=dt, device=dev)
                for j, t in enumerate(present):
                    B[offs[t]:offs[t] + sizes[t], j * r:(j + 1) * r] = col(targets[t]["B"])[starts[t]:starts[t] + sizes[t]]
                layers[(li, "qkv_proj")] = LoRALayerWeights(_pad_rank(A, 0), _pad_rank(B, 1))
            # ---- packed gate | up (column-parallel) ----
            present = [t for t in ("gate_proj", "up_proj") if t in targets]
            if present and layer.gate_up_proj is not None:
                I = layer.gate_up_proj.out_per_rank // 2
                A = torch.cat([col(targets[t]["A"]) for t in present], dim=0)
                B = torch.zeros(2 * I, len(present) * r, dtype=dt, device=dev)
                for j, t in enumerate(present):
                    o = 0 if t == "gate_proj" else I
                    B[o:o + I, j * r:(j + 1) * r] = col(targets[t]["B"])[rank * I:(rank + 1) * I]
                layers[(li, "gate_up_proj")] = LoRALayerWeights(_pad_rank(A, 0), _pad_rank(B, 1))
            # ---- row-parallel layers ----
            for t, mod in (("o_proj", layer.o_proj), ("down_proj", layer.down_proj)):
                if t in targets and mod is not None:
                    k = mod.in_per_rank
                    A = col(targets[t]["A"])[:, rank * k:(rank + 1) * k]
                    layers[(li, t)] = LoRALayerWeights(_pad_rank(A, 0), _pad_rank(col(targets[t]["B"]), 1))
        return LoRAAdapter(name, r, scaling, layers)


class LoRAManager:
    """Adapters resident on this worker and the token -> adapter map of the step being executed."""

    def __init__(self, model, max_loras: int = 8):
        self.model = model
        self.max_loras = max_loras
        self.adapters: dict[int, LoRAAdapter] = {}
        self._order: list[int] = []           # least recently used first
        self._row_adapter: Optional[torch.Tensor] = None
        self._segments_cache: dict = {}
        self.active = False

    def ensure_loaded(self, req: LoRARequest) -> None:
        if req.lora_int_id in self.adapters:
            self._order.remove(req.lora_int_id)
            self._order.append(req.lora_int_id)
            return
        if len(self.adapters) >= self.max_loras:
            victim = self._order.pop(0)
            del self.adapters[victim]
        self.adapters[req.lora_int_id] = LoRAAdapter.load(req.lora_path, self.model, req.lora_name)
        self._order.append(req.lora_int_id)

    def add_adapter(self, lora_int_id: int, adapter: LoRAAdapter) -> None:
        self.adapters[lora_int_id] = adapter
        if lora_int_id not in self._order:
            self._order.append(lora_int_id)

    def set_batch(self, row_adapter_ids: list[int]) -> None:
        """``row_adapter_ids[i]``: adapter id of token row i of the step (0 = none)."""
        self.active = any(a != 0 for a in row_adapter_ids)
        self._segments_cache = {}
        self._row_adapter = torch.tensor(row_adapter_ids, dtype=torch.int64) if self.active else None

    def segments(self, row0: int, n: int, device) -> list:
        """[(adapter, row indices relative to row0)] for the adapters used by rows [row0, row0 + n)."""
        if not self.active or n == 0:
            return []
        key = (row0, n)
        segs = self._segments_cache.get(key)
        if segs is None:
            ids = self._row_adapter[row0:row0 + n]
            segs = []
            for a in ids.unique().tolist():
                if a != 0:
                    segs.append((self.adapters[a], (ids == a).nonzero().flatten().to(device)))
            self._segments_cache[key] = segs
        return segs

    @staticmethod
    def apply(segs: list, layer_idx: int, which: str, x: torch.Tensor, out: torch.Tensor) -> None:
        """out[rows] += scaling * (x[rows] @ A^T) @ B^T for every adapter of the step that targets this layer."""
        for adapter, idx in segs:
            w = adapter.layers.get((layer_idx, which))
            if w is None:
                continue
            xs = x.index_select(0, idx).contiguous()
            t = ops.gemm(xs, w.A)
            delta = ops.gemm(t, w.B)
            out.index_add_(0, idx, delta, alpha=adapter.scaling)
