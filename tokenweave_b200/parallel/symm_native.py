"""The package's own symmetric-memory provider (``TW_SYMM_PROVIDER=native``).

Driver calls live in ``csrc/symm_heap.cu`` (CUDA virtual-memory-management API); this module moves the
exported POSIX file descriptors between the ranks of the node over Unix sockets (``SCM_RIGHTS``) and
sequences the steps with the host-side gloo group:

1. every rank creates a physical allocation (data + signal pad), maps it and exports it;
2. all-to-all exchange of the descriptors; every rank maps every peer's allocation;
3. rank 0 creates the multicast object and hands its descriptor to all ranks; every rank joins the
   multicast team, and after a barrier binds its allocation and maps the multicast address range.

``close()`` undoes it in the reverse order behind a barrier, so no rank unbinds while another still
uses the multicast address.
"""
from __future__ import annotations

import ctypes as C
import os
import socket
import threading
import uuid
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _native
from .state import TPState
from .symm_mem import SIGNAL_PAD_WORDS_NEEDED, SymmetricBuffer

_u64p = C.POINTER(C.c_ulonglong)
_bound = False


def _bind():
    global _bound
    lib = _native.load()
    if _bound:
        return lib
    u64, i32 = C.c_ulonglong, C.c_int
    sigs = {
        "tw_symm_granularity": [i32, i32, _u64p],
        "tw_symm_multicast_supported": [i32],
        "tw_symm_alloc_local": [i32, u64, _u64p, _u64p, C.POINTER(i32)],
        "tw_symm_import_peer": [i32, i32, u64, _u64p, _u64p],
        "tw_symm_multicast_create": [i32, u64, _u64p, C.POINTER(i32)],
        "tw_symm_multicast_import": [i32, _u64p],
        "tw_symm_multicast_add_device": [u64, i32],
        "tw_symm_multicast_bind_map": [u64, u64, i32, u64, _u64p],
        "tw_symm_release": [u64, u64, u64, i32, i32],
    }
    for name, argtypes in sigs.items():
        fn = getattr(lib, name)
        fn.restype = C.c_int
        fn.argtypes = argtypes
    _bound = True
    return lib


def _check(lib, rc: int, what: str) -> None:
    if rc != 0:
        msg = lib.tw_last_error()
        raise RuntimeError(f"{what}: {msg.decode() if msg else 'failed'}")


class _RawCudaMemory:
    """Exposes a raw device allocation to PyTorch through ``__cuda_array_interface__`` (zero copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def _exchange_fds(tp: TPState, my_fd: Optional[int], tag: str, root_only: bool = False) -> dict[int, int]:
    """All-to-all (or root-to-all) hand-over of one file descriptor per rank over Unix sockets."""
    base = [None]
    if tp.rank == 0:
        base[0] = os.path.join("/tmp", f"tw_symm_{uuid.uuid4().hex[:12]}_{tag}")
    dist.broadcast_object_list(base, src=dist.get_global_rank(tp.cpu_group, 0), group=tp.cpu_group)
    path = lambda r: f"{base[0]}_{r}.sock"
    expect = (0 if tp.rank == 0 else 1) if root_only else tp.world_size - 1
    got: dict[int, int] = {}
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    try:
        os.unlink(path(tp.rank))
    except FileNotFoundError:
        pass
    server.bind(path(tp.rank))
    server.listen(tp.world_size)
    server.settimeout(60)

    def accept_all():
        for _ in range(expect):
            conn, _ = server.accept()
            with conn:
                msg, fds, _, _ = socket.recv_fds(conn, 16, 1)
                got[int(msg.decode())] = fds[0]

    t = threading.Thread(target=accept_all, daemon=True)
    t.start()
    dist.barrier(group=tp.cpu_group)                 # every server is listening
    senders = [0] if root_only else range(tp.world_size)
    if tp.rank in senders:
        for peer in range(tp.world_size):
            if peer == tp.rank:
                continue
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                c.settimeout(60)
                c.connect(path(peer))
                socket.send_fds(c, [str(tp.rank).encode()], [my_fd])
    t.join(90)
    if t.is_alive() or len(got) != expect:
        raise RuntimeError(f"rank {tp.rank}: received {len(got)} of {expect} file descriptors ({tag})")
    dist.barrier(group=tp.cpu_group)
    server.close()
    try:
        os.unlink(path(tp.rank))
    except FileNotFoundError:
        pass
    return got


class NativeSymmHandle:
    def __init__(self):
        self.lib = None
        self.tp: Optional[TPState] = None
        self.size = 0
        self.local = (0, 0)                       # (handle, va)
        self.peers: dict[int, tuple[int, int]] = {}
        self.mc = (0, 0)
        self.pad_offset = 0
        self.pad_tensor: Optional[torch.Tensor] = None
        self.closed = False

    def reset_signal_pad(self) -> None:
        self.pad_tensor.zero_()

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        tp, lib = self.tp, self.lib
        torch.cuda.synchronize()
        dist.barrier(group=tp.cpu_group)          # nobody is inside a kernel that touches the mappings
        dev = tp.device.index
        if self.mc[0]:
            lib.tw_symm_release(self.mc[1], self.size, self.mc[0], 1, dev)
        dist.barrier(group=tp.cpu_group)
        for r, (h, va) in self.peers.items():
            lib.tw_symm_release(va, self.size, h, 0, dev)
        lib.tw_symm_release(self.local[1], self.size, self.local[0], 0, dev)


def create_native_buffer(rows: int, cols: int, dtype: torch.dtype, tp: TPState, allow_multicast: bool) -> SymmetricBuffer:
    lib = _bind()
    dev = tp.device.index
    torch.cuda.set_device(dev)
    torch.zeros(1, device=tp.device)              # make sure the primary context exists
    gran = C.c_ulonglong(0)
    _check(lib, lib.tw_symm_granularity(dev, tp.world_size, C.byref(gran)), "granularity")
    data_bytes = rows * cols * dtype.itemsize
    pad_offset = (data_bytes + 1023) // 1024 * 1024
    pad_bytes = SIGNAL_PAD_WORDS_NEEDED * 4
    size = (pad_offset + pad_bytes + gran.value - 1) // gran.value * gran.value

    h = NativeSymmHandle()
    h.lib, h.tp, h.size, h.pad_offset = lib, tp, size, pad_offset
    handle, va, fd = C.c_ulonglong(0), C.c_ulonglong(0), C.c_int(-1)
    _check(lib, lib.tw_symm_alloc_local(dev, size, C.byref(handle), C.byref(va), C.byref(fd)), "alloc_local")
    h.local = (handle.value, va.value)
    raw = torch.as_tensor(_RawCudaMemory(va.value, size), device=tp.device)
    raw.zero_()
    torch.cuda.synchronize()

    fds = _exchange_fds(tp, fd.value, "mem")
    for r, pfd in fds.items():
        ph, pva = C.c_ulonglong(0), C.c_ulonglong(0)
        _check(lib, lib.tw_symm_import_peer(dev, pfd, size, C.byref(ph), C.byref(pva)), f"import_peer({r})")
        h.peers[r] = (ph.value, pva.value)
        os.close(pfd)
    os.close(fd.value)

    mc_va = 0
    want_mc = allow_multicast and bool(lib.tw_symm_multicast_supported(dev))
    flags = [None] * tp.world_size
    dist.all_gather_object(flags, want_mc, group=tp.cpu_group)
    if all(flags):
        mch, mcfd = C.c_ulonglong(0), C.c_int(-1)
        if tp.rank == 0:
            _check(lib, lib.tw_symm_multicast_create(tp.world_size, size, C.byref(mch), C.byref(mcfd)), "multicast_create")
        got = _exchange_fds(tp, mcfd.value if tp.rank == 0 else None, "mc", root_only=True)
        if tp.rank != 0:
            _check(lib, lib.tw_symm_multicast_import(got[0], C.byref(mch)), "multicast_import")
            os.close(got[0])
        else:
            os.close(mcfd.value)
        _check(lib, lib.tw_symm_multicast_add_device(mch.value, dev), "multicast_add_device")
        dist.barrier(group=tp.cpu_group)          # the whole team has joined
        out = C.c_ulonglong(0)
        _check(lib, lib.tw_symm_multicast_bind_map(mch.value, h.local[0], dev, size, C.byref(out)), "multicast_bind_map")
        mc_va = out.value
        h.mc = (mch.value, mc_va)
        dist.barrier(group=tp.cpu_group)

    bases = [h.local[1] if r == tp.rank else h.peers[r][1] for r in range(tp.world_size)]
    peer_ptrs = torch.tensor(bases, dtype=torch.int64, device=tp.device)
    pad_ptrs = torch.tensor([b + pad_offset for b in bases], dtype=torch.int64, device=tp.device)
    data = raw[:data_bytes].view(dtype).view(rows, cols)
    h.pad_tensor = raw[pad_offset:pad_offset + pad_bytes].view(torch.int32)
    h._keep = (raw, peer_ptrs, pad_ptrs)
    torch.cuda.synchronize()
    dist.barrier(group=tp.cpu_group)
    return SymmetricBuffer(data, tp.rank, tp.world_size, mc_va, peer_ptrs.data_ptr(), pad_ptrs.data_ptr(), "native", h,
                           SIGNAL_PAD_WORDS_NEEDED, tuple(bases))
