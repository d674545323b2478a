"""Sleep mode on the VMM allocator of ``csrc/vmm_allocator.cu``.

Allocations made inside :meth:`SleepAllocator.use_pool` come from a ``torch.cuda.MemPool`` whose
backing allocator reserves a virtual range and maps physical memory behind it; :meth:`sleep` releases
the physical memory of every such allocation (saving the tagged ones to pinned host memory) and
:meth:`wake_up` maps fresh memory at the same addresses, so every tensor — and every CUDA graph that
captured its address — stays valid. Counterpart of vllm/device_allocator/cumem.py:1-280
(``CuMemAllocator.use_memory_pool / sleep / wake_up``) with the bookkeeping in the native library.
"""
from __future__ import annotations

import contextlib
import ctypes as C
from typing import Iterable, Optional

import torch

from ..ops import _native

TAG_WEIGHTS = 1
TAG_KV_CACHE = 2
TAG_OTHER = 3


class SleepAllocator:
    _instance: Optional["SleepAllocator"] = None

    @classmethod
    def get(cls) -> "SleepAllocator":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def __init__(self):
        self.lib = _native.load()
        self.lib.tw_vmm_bytes.restype = C.c_longlong
        self.lib.tw_vmm_bytes.argtypes = [C.c_int]
        for name, args in (("tw_vmm_set_tag", [C.c_int]), ("tw_vmm_sleep", [C.c_uint]), ("tw_vmm_wake", [C.c_uint])):
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = C.c_int, args
        self._pluggable = torch.cuda.memory.CUDAPluggableAllocator(str(_native.lib_path()), "tw_vmm_malloc", "tw_vmm_free")
        self._pools: dict[int, torch.cuda.MemPool] = {}
        self.asleep = False

    @contextlib.contextmanager
    def use_pool(self, tag: int):
        """Route the CUDA allocations of the enclosed block to the sleep-capable pool of ``tag``."""
        pool = self._pools.get(tag)
        if pool is None:
            pool = self._pools[tag] = torch.cuda.MemPool(self._pluggable.allocator())
        self.lib.tw_vmm_set_tag(tag)
        try:
            with torch.cuda.use_mem_pool(pool):
                yield
        finally:
            self.lib.tw_vmm_set_tag(0)

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            msg = self.lib.tw_last_error()
            raise RuntimeError(f"{what} failed: {msg.decode() if msg else 'unknown error'}")

    def sleep(self, offload_tags: Iterable[int] = (TAG_WEIGHTS,)) -> None:
        """Release all device memory of the pools; contents of ``offload_tags`` move to pinned host memory,
        everything else is discarded."""
        torch.cuda.synchronize()
        mask = 0
        for t in offload_tags:
            mask |= 1 << t
        self._check(self.lib.tw_vmm_sleep(mask), "vmm sleep")
        self.asleep = True

    def wake_up(self, tags: Optional[Iterable[int]] = None) -> None:
        mask = 0xFFFFFFFF
        if tags is not None:
            mask = 0
            for t in tags:
                mask |= 1 << t
        self._check(self.lib.tw_vmm_wake(mask), "vmm wake")
        torch.cuda.synchronize()
        self.asleep = self.mapped_bytes() < self.reserved_bytes()

    def mapped_bytes(self) -> int:
        return int(self.lib.tw_vmm_bytes(0))

    def reserved_bytes(self) -> int:
        return int(self.lib.tw_vmm_bytes(1))

    def host_bytes(self) -> int:
        return int(self.lib.tw_vmm_bytes(2))
