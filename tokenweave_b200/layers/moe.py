"""Mixture-of-experts MLP with tensor-sharded experts (Mixtral).

Counterpart of vllm/model_executor/layers/fused_moe/layer.py:840-895 and fused_moe.py:1230-1426. Expert
weights are ``w13 = [E, 2*I/tp, H]`` (w1 = gate rows first, w3 = up rows second) and
``w2 = [E, H, I/tp]``; the router gate is replicated. The output is this rank's partial sum written in
place into the caller's rows of the symmetric buffer (no all-reduce here).

GPU pipeline: fused gate-GEMV/softmax/top-k -> align (pad every expert to 128 rows) -> scatter rows into
expert order -> grouped tcgen05 GEMM with SwiGLU epilogue -> grouped GEMM scaled by the routing weight
-> deterministic top-k combine.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..ops import reference
from ..parallel.state import get_tp

TILE_ROWS = 128          # rows every expert's group is padded to ...
TILE_ROWS_PAIR = 256     # ... or, once an expert gets 512 rows or more on average, this: the groups then run on
                         # CTA pairs (256-row tcgen05 tiles), which more than pays for the extra padding


class FusedMoE(nn.Module):
    def __init__(self, num_experts: int, top_k: int, hidden: int, intermediate: int, *, dtype, device,
                 renormalize: bool = True, expert_parallel: bool = False):
        super().__init__()
        tp = get_tp()
        self.num_experts_global, self.top_k, self.hidden = num_experts, top_k, hidden
        self.expert_parallel = expert_parallel and tp.world_size > 1
        if self.expert_parallel:
            # whole experts per rank (vllm/model_executor/layers/fused_moe/layer.py:332-374 ``determine_expert_map``):
            # every rank routes all tokens, runs the pairs that hit its experts and contributes a partial
            # sum, so the collective that follows is the same reduce-scatter as with tensor-sharded experts
            assert num_experts % tp.world_size == 0
            self.E = num_experts // tp.world_size
            self.expert_base = tp.rank * self.E
            self.inter_per_rank = intermediate
        else:
            assert intermediate % tp.world_size == 0
            self.E, self.expert_base = num_experts, 0
            self.inter_per_rank = intermediate // tp.world_size
        self.renormalize = renormalize
        I = self.inter_per_rank
        self.gate = nn.Parameter(torch.empty(num_experts, hidden, dtype=dtype, device=device), requires_grad=False)
        self.w13 = nn.Parameter(torch.empty(self.E, 2 * I, hidden, dtype=dtype, device=device), requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(self.E, hidden, I, dtype=dtype, device=device), requires_grad=False)
        self._ws_tokens = 0
        self._ws = None
        self.pair_tiles = True      # False: 128-row groups at every size (tests, comparisons)

    # ---- checkpoint loading (experts.{e}.w1/w2/w3 -> w13 / w2) ----
    def load_expert_weight(self, expert: int, which: str, loaded: torch.Tensor) -> None:
        tp = get_tp()
        I = self.inter_per_rank
        if self.expert_parallel:
            expert -= self.expert_base
            if not 0 <= expert < self.E:
                return                                  # another rank's expert
            dst = {"w1": self.w13.data[expert, :I], "w3": self.w13.data[expert, I:], "w2": self.w2.data[expert]}
            if which not in dst:
                raise KeyError(which)
            dst[which].copy_(loaded)
            return
        if which == "w1":
            self.w13.data[expert, :I].copy_(loaded.narrow(0, tp.rank * I, I))
        elif which == "w3":
            self.w13.data[expert, I:].copy_(loaded.narrow(0, tp.rank * I, I))
        elif which == "w2":
            self.w2.data[expert].copy_(loaded.narrow(1, tp.rank * I, I))
        else:
            raise KeyError(which)

    def _workspace(self, T: int, device):
        if self._ws is None or self._ws_tokens < T:
            n_pairs = T * self.top_k
            max_rows = (n_pairs + self.E * (TILE_ROWS_PAIR - 1) + TILE_ROWS_PAIR - 1) // TILE_ROWS_PAIR * TILE_ROWS_PAIR
            max_tiles = max_rows // TILE_ROWS
            i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=device)
            dt = self.w13.dtype
            self._ws = dict(
                offsets=i32(self.E + 1), cursor=i32(self.E), tile_expert=i32(max_tiles), meta=i32(2),
                a_sorted=torch.zeros(max_rows, self.hidden, dtype=dt, device=device),
                act=torch.zeros(max_rows, self.inter_per_rank, dtype=dt, device=device),
                y=torch.zeros(max_rows, self.hidden, dtype=dt, device=device),
                row_scale=torch.zeros(max_rows, dtype=torch.float32, device=device),
                sorted_pos=i32(T, self.top_k))
            self._ws_tokens = T
        return self._ws

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
        T, H = x.shape
        if out is None:
            out = torch.empty_like(x)
        if T == 0:
            return out
        topk_w, topk_ids, _ = ops.moe_router(x, self.gate, self.top_k, self.renormalize)
        if self.expert_parallel:
            # local expert index, or -1 for pairs that belong to another rank (align / scatter / combine skip them)
            local = topk_ids - self.expert_base
            topk_ids = torch.where((local >= 0) & (local < self.E), local, torch.full_like(local, -1))
        if not x.is_cuda:
            out.copy_(reference.moe_experts(x, self.w13, self.w2, topk_w, topk_ids))
            return out
        ws = self._workspace(T, x.device)
        E, I = self.E, self.inter_per_rank
        tile_rows = TILE_ROWS_PAIR if T * self.top_k >= 512 * E and self.pair_tiles else TILE_ROWS
        n_rows = (T * self.top_k + E * (tile_rows - 1) + tile_rows - 1) // tile_rows * tile_rows
        tile_expert = ws["tile_expert"][: n_rows // tile_rows]
        ops.moe_align(topk_ids, E, tile_rows, ws["offsets"], ws["cursor"], tile_expert, ws["meta"])
        sorted_pos = ws["sorted_pos"][:T]
        ops.moe_scatter(x, topk_ids, topk_w, ws["offsets"], ws["cursor"], ws["a_sorted"], ws["row_scale"],
                        sorted_pos, E)
        a = ws["a_sorted"][:n_rows]
        act = ops.gemm(a, self.w13.view(E * 2 * I, H), out=ws["act"][:n_rows], swiglu=True, tile_expert=tile_expert,
                       num_m_tiles=ws["meta"][:1], n_per_expert=2 * I, max_ctas=max_ctas, tile_rows=tile_rows)
        y = ops.gemm(act, self.w2.view(E * H, I), out=ws["y"][:n_rows], row_scale=ws["row_scale"],
                     tile_expert=tile_expert, num_m_tiles=ws["meta"][:1], n_per_expert=H, max_ctas=max_ctas,
                     tile_rows=tile_rows)
        ops.moe_combine(y, sorted_pos, out, self.top_k)
        return out
