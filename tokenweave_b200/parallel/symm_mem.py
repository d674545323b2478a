"""Symmetric memory: one buffer of identical size on every TP rank, reachable from every GPU through
peer pointers and (where NVSwitch offers NVLS) one multicast address, plus per-rank signal pads for
the in-kernel barrier.

Reference: ``torch.distributed._symmetric_memory.empty`` + ``rendezvous`` at
vllm/model_executor/models/llama.py:437-441; handle fields used by its kernels: ``multicast_ptr``,
``signal_pad_ptrs_dev``. Providers here:

* ``torch``  : PyTorch's symmetric-memory rendezvous (CUDA VMM + multicast underneath).
* ``native`` : the package's own allocator (``csrc/symm_heap.cu``: cuMemCreate, POSIX fd exchange over
               a Unix socket, cuMulticast* binding), selected with ``TW_SYMM_PROVIDER=native``.
* ``local``  : world size 1 or CPU: a plain tensor, no peers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import envs
from .state import TPState, get_tp

SIGNAL_PAD_WORDS_NEEDED = 2 * 128 * 8 + 64   # two alternating sets of barrier flags (128 CTAs x 8 ranks each), plus spare flags


@dataclass
class SymmetricBuffer:
    tensor: torch.Tensor                   # this rank's copy, viewed as [rows, cols]
    rank: int
    world: int
    multicast_ptr: int = 0                 # 0: no NVLS mapping, kernels use peer loads/stores
    peer_ptrs_dev: int = 0                 # device address of an array of `world` buffer pointers
    signal_pads_dev: int = 0               # device address of an array of `world` signal-pad pointers
    provider: str = "local"
    handle: object = None                  # keeps the provider's allocation alive
    signal_pad_words: int = 0
    peer_ptrs_host: tuple = ()             # the same `world` buffer addresses, on the host

    def pointer_table(self, byte_offset: int) -> torch.Tensor:
        """Device array of `world` pointers: every rank's copy of the buffer plus ``byte_offset``."""
        return torch.tensor([p + byte_offset for p in self.peer_ptrs_host], dtype=torch.int64, device=self.tensor.device)

    @property
    def base_ptr(self) -> int:
        return self.tensor.data_ptr()

    def byte_offset(self, view: torch.Tensor) -> int:
        """Offset of a view of ``tensor`` from the start of the buffer (same on every rank)."""
        off = view.data_ptr() - self.tensor.data_ptr()
        if off < 0 or off + view.numel() * view.element_size() > self.tensor.numel() * self.tensor.element_size():
            raise ValueError("tensor is not a view of this symmetric buffer")
        return off

    @property
    def has_multicast(self) -> bool:
        return self.multicast_ptr != 0

    def close(self) -> None:
        """Collective tear-down (native provider: unbind / unmap behind a barrier)."""
        if self.provider == "native" and self.handle is not None:
            self.handle.close()
        self.handle = None

    def reset_signal_pads(self) -> None:
        """Zero this rank's signal pad (after a kernel reported a peer timeout)."""
        if self.provider == "torch" and self.handle is not None:
            pad = self.handle.get_signal_pad(self.rank, dtype=torch.int32)
            pad.zero_()
        elif self.provider == "native" and self.handle is not None:
            self.handle.reset_signal_pad()


def create_symmetric_buffer(rows: int, cols: int, dtype: torch.dtype, tp: Optional[TPState] = None,
                            provider: Optional[str] = None, allow_multicast: bool = True) -> SymmetricBuffer:
    tp = tp or get_tp()
    if tp.world_size == 1 or tp.device.type != "cuda":
        t = torch.zeros(rows, cols, dtype=dtype, device=tp.device)
        return SymmetricBuffer(t, tp.rank, tp.world_size)
    provider = provider or envs.TW_SYMM_PROVIDER
    if provider == "native":
        from .symm_native import create_native_buffer
        return create_native_buffer(rows, cols, dtype, tp, allow_multicast and not envs.TW_DISABLE_NVLS)
    return _create_torch_buffer(rows, cols, dtype, tp, allow_multicast and not envs.TW_DISABLE_NVLS)


def _create_torch_buffer(rows: int, cols: int, dtype: torch.dtype, tp: TPState, allow_multicast: bool) -> SymmetricBuffer:
    import torch.distributed._symmetric_memory as symm_mem
    try:
        if symm_mem.get_signal_pad_size() < SIGNAL_PAD_WORDS_NEEDED * 4:
            symm_mem.set_signal_pad_size(SIGNAL_PAD_WORDS_NEEDED * 4)
    except Exception:
        pass
    t = symm_mem.empty(rows, cols, dtype=dtype, device=tp.device)
    hdl = symm_mem.rendezvous(t, tp.group.group_name if hasattr(tp.group, "group_name") else tp.group)
    t.zero_()
    mc = int(hdl.multicast_ptr) if allow_multicast and hdl.multicast_ptr else 0
    buf = SymmetricBuffer(t, tp.rank, tp.world_size, mc, int(hdl.buffer_ptrs_dev), int(hdl.signal_pad_ptrs_dev),
                          "torch", hdl, int(hdl.signal_pad_size) // 4, tuple(int(x) for x in hdl.buffer_ptrs))
    torch.cuda.synchronize()
    hdl.barrier(channel=0)
    return buf
