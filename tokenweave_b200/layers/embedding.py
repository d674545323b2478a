"""Token embedding and LM head.

The embedding table is replicated on every rank by default: at 180 GB of HBM per GPU its 2 GB buy out
the all-reduce the reference pays after a vocab-parallel lookup
(vllm/model_executor/layers/vocab_parallel_embedding.py:407-485). The vocab-parallel layout is kept as
an option (``parallel=True``): rows outside this rank's vocabulary slice come out as zeros and the
partial result is reduced by the same fused collective as every other layer output (with a zero
residual), so split 1's reduction overlaps split 0's attention exactly as in the reference.
The LM head is always vocab-parallel (vocabulary padded to a multiple of 64 * tp); logits are
all-gathered (logits_processor.py:87-118 gathers to rank 0; here every rank keeps them so that SPMD
ranks sample identically).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..parallel.state import get_tp


def pad_vocab(vocab: int, multiple: int) -> int:
    return (vocab + multiple - 1) // multiple * multiple


class VocabEmbedding(nn.Module):
    def __init__(self, vocab_size: int, hidden: int, parallel: bool = False, *, dtype, device):
        super().__init__()
        tp = get_tp()
        self.vocab_size = vocab_size
        self.parallel = parallel and tp.world_size > 1
        if self.parallel:
            padded = pad_vocab(vocab_size, 64 * tp.world_size)
            self.per_rank = padded // tp.world_size
            self.vocab_start = tp.rank * self.per_rank
            rows = self.per_rank
        else:
            self.vocab_start, rows = 0, vocab_size
            self.per_rank = rows
        self.weight = nn.Parameter(torch.zeros(rows, hidden, dtype=dtype, device=device), requires_grad=False)

    def forward(self, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.embedding(ids, self.weight, out=out, vocab_start=self.vocab_start,
                             vocab_end=self.vocab_start + self.per_rank)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        if not self.parallel:
            param.data[: loaded.shape[0]].copy_(loaded)
            return
        lo = self.vocab_start
        hi = min(lo + self.per_rank, loaded.shape[0])
        if hi > lo:
            param.data[: hi - lo].copy_(loaded[lo:hi])


class ParallelLMHead(nn.Module):
    def __init__(self, vocab_size: int, hidden: int, *, dtype, device):
        super().__init__()
        tp = get_tp()
        self.vocab_size = vocab_size
        self.padded = pad_vocab(vocab_size, 64 * tp.world_size)
        self.per_rank = self.padded // tp.world_size
        self.vocab_start = tp.rank * self.per_rank
        self.weight = nn.Parameter(torch.zeros(self.per_rank, hidden, dtype=dtype, device=device),
                                   requires_grad=False)
        self.comm = None       # TPCommunicator of the runtime: its private NCCL communicator gathers the logits

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        """fp32 logits ``[rows, vocab_size]`` on every rank."""
        tp = get_tp()
        local = ops.gemm(hidden, self.weight)
        if tp.world_size > 1:
            rows, cols = local.shape
            gathered = torch.empty(tp.world_size * rows, cols, dtype=local.dtype, device=local.device)
            if self.comm is not None:
                self.comm.nccl_all_gather(gathered.view(-1), local.contiguous().view(-1))
            else:
                dist.all_gather_into_tensor(gathered, local.contiguous(), group=tp.group)
            local = gathered.view(tp.world_size, rows, cols).permute(1, 0, 2).reshape(rows, -1)
        return local[:, : self.vocab_size].float()

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        lo = self.vocab_start
        hi = min(lo + self.per_rank, loaded.shape[0])
        if hi > lo:
            param.data[: hi - lo].copy_(loaded[lo:hi])
