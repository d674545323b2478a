"""Peer-to-peer all-reduce with the size policy of a classic custom all-reduce: one-shot (every rank
pulls the whole message from every peer) for small messages, two-shot (reduce-scatter + all-gather over
peer pointers) above the threshold, NCCL beyond the maximum registered size.

Counterpart of csrc/custom_all_reduce.cuh:296-364,558-589 and
vllm/distributed/device_communicators/custom_all_reduce.py:48-301 (8 MB maximum, world size in
{2, 4, 6, 8}, one-shot below 512 KiB for world <= 4 and below 256 KiB for world <= 8). It is the baseline
the TokenWeave runs switch off (``disable_custom_all_reduce=True``); kept for comparisons."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .comm import TPCommunicator
from .symm_mem import create_symmetric_buffer

MAX_BYTES = 8 << 20


class CustomAllReduce:
    def __init__(self, tp, max_bytes: int = MAX_BYTES):
        if tp.world_size not in (2, 4, 6, 8):
            raise ValueError("custom all-reduce supports world sizes 2, 4, 6 and 8")
        self.tp = tp
        self.max_bytes = max_bytes
        self.buf = create_symmetric_buffer(max_bytes // 2, 1, torch.bfloat16, tp, allow_multicast=False)
        self.comm = TPCommunicator(self.buf, tp, transport="p2p")
        self.out = torch.empty(max_bytes // 2, dtype=torch.bfloat16, device=tp.device)

    def should_use(self, x: torch.Tensor) -> bool:
        return x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() * 2 <= self.max_bytes and (x.numel() * 2) % (16 * self.tp.world_size) == 0

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Returns the reduced tensor (a view of an internal buffer, valid until the next call)."""
        if not self.should_use(x):
            dist.all_reduce(x, group=self.tp.group)
            return x
        n = x.numel()
        nbytes = n * 2
        stage = self.buf.tensor.view(-1)[:n]
        stage.copy_(x.view(-1))
        w = self.tp.world_size
        one_shot = (w <= 4 and nbytes < 512 * 1024) or (w <= 8 and nbytes < 256 * 1024)
        if one_shot:
            self.comm.oneshot_all_reduce(stage, self.out[:n])
            return self.out[:n].view_as(x)
        self.comm.all_reduce_(stage, max_ctas=36)
        return stage.view_as(x)
