"""NCCL through ctypes: a communicator of its own, next to (not inside) ``torch.distributed``.

Counterpart of vllm/distributed/device_communicators/pynccl.py:109-217 and pynccl_wrapper.py: the reference
keeps a private NCCL communicator so that collectives can be captured in CUDA graphs and issued on a chosen
stream without going through the process-group layer. Here it is the library-only baseline of the
``baseline_nccl`` schedule and of ``artifact/collectives_bench.py``; the product path does its collectives
inside its own kernels (``csrc/comm_fused.cu``). The unique id travels over any object broadcast the caller
provides (the gloo twin group, a :class:`~tokenweave_b200.parallel.store_group.StoreGroup`).

Loading the library and reading its version work anywhere; communicators need GPUs.
"""
from __future__ import annotations

import ctypes
import glob
import os
from typing import Callable, Optional

import torch

ncclResult_t = ctypes.c_int
ncclComm_t = ctypes.c_void_p


class ncclUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


# ncclDataType_t / ncclRedOp_t of nccl.h
_DTYPES = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
           torch.float64: 8, torch.bfloat16: 9}
_OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}


def find_library() -> str:
    """``TW_NCCL_SO_PATH``, else the libnccl that ships with torch, else the system's."""
    env = os.environ.get("TW_NCCL_SO_PATH")
    if env:
        return env
    bundled = sorted(glob.glob(os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "nccl", "lib", "libnccl.so*")))
    return bundled[0] if bundled else "libnccl.so.2"


class NCCLLibrary:
    _SIGNATURES = {
        "ncclGetErrorString": (ctypes.c_char_p, [ncclResult_t]),
        "ncclGetVersion": (ncclResult_t, [ctypes.POINTER(ctypes.c_int)]),
        "ncclGetUniqueId": (ncclResult_t, [ctypes.POINTER(ncclUniqueId)]),
        "ncclCommInitRank": (ncclResult_t, [ctypes.POINTER(ncclComm_t), ctypes.c_int, ncclUniqueId, ctypes.c_int]),
        "ncclAllReduce": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                        ncclComm_t, ctypes.c_void_p]),
        "ncclAllGather": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ncclComm_t,
                                        ctypes.c_void_p]),
        "ncclReduceScatter": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                            ctypes.c_int, ncclComm_t, ctypes.c_void_p]),
        "ncclBroadcast": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                        ncclComm_t, ctypes.c_void_p]),
        "ncclSend": (ncclResult_t, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t,
                                   ctypes.c_void_p]),
        "ncclRecv": (ncclResult_t, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t,
                                   ctypes.c_void_p]),
        "ncclCommDestroy": (ncclResult_t, [ncclComm_t]),
    }

    def __init__(self, path: Optional[str] = None):
        self.path = path or find_library()
        self.lib = ctypes.CDLL(self.path)
        for name, (res, args) in self._SIGNATURES.items():
            f = getattr(self.lib, name)
            f.restype, f.argtypes = res, args

    def check(self, result: int) -> None:
        if result != 0:
            raise RuntimeError(f"NCCL error {result}: {self.lib.ncclGetErrorString(result).decode()}")

    def version(self) -> str:
        v = ctypes.c_int()
        self.check(self.lib.ncclGetVersion(ctypes.byref(v)))
        major, rest = divmod(v.value, 10000)
        minor, patch = divmod(rest, 100)
        return f"{major}.{minor}.{patch}"


class NcclCommunicator:
    """``broadcast_obj(obj, src)`` must deliver rank 0's unique id to every rank (any control-plane group)."""

    def __init__(self, rank: int, world_size: int, device: torch.device, broadcast_obj: Callable,
                 library: Optional[NCCLLibrary] = None):
        self.rank, self.world_size, self.device = rank, world_size, torch.device(device)
        self.nccl = library or NCCLLibrary()
        uid = ncclUniqueId()
        if rank == 0:
            self.nccl.check(self.nccl.lib.ncclGetUniqueId(ctypes.byref(uid)))
        raw = broadcast_obj(bytes(uid.internal) if rank == 0 else None, 0)
        ctypes.memmove(ctypes.byref(uid), raw, 128)
        self.comm = ncclComm_t()
        with torch.cuda.device(self.device):
            self.nccl.check(self.nccl.lib.ncclCommInitRank(ctypes.byref(self.comm), world_size, uid, rank))
            warm = torch.zeros(1, device=self.device)      # the first collective builds the rings / trees
            self.all_reduce(warm)
            torch.cuda.current_stream().synchronize()

    def _stream(self, stream) -> ctypes.c_void_p:
        return ctypes.c_void_p((stream or torch.cuda.current_stream(self.device)).cuda_stream)

    def all_reduce(self, t: torch.Tensor, op: str = "sum", out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        out = t if out is None else out
        self.nccl.check(self.nccl.lib.ncclAllReduce(t.data_ptr(), out.data_ptr(), t.numel(), _DTYPES[t.dtype], _OPS[op],
                                                    self.comm, self._stream(stream)))
        return out

    def all_gather(self, out: torch.Tensor, t: torch.Tensor, stream=None) -> torch.Tensor:
        self.nccl.check(self.nccl.lib.ncclAllGather(t.data_ptr(), out.data_ptr(), t.numel(), _DTYPES[t.dtype], self.comm,
                                                    self._stream(stream)))
        return out

    def reduce_scatter(self, out: torch.Tensor, t: torch.Tensor, op: str = "sum", stream=None) -> torch.Tensor:
        self.nccl.check(self.nccl.lib.ncclReduceScatter(t.data_ptr(), out.data_ptr(), out.numel(), _DTYPES[t.dtype],
                                                        _OPS[op], self.comm, self._stream(stream)))
        return out

    def broadcast(self, t: torch.Tensor, src: int, stream=None) -> torch.Tensor:
        self.nccl.check(self.nccl.lib.ncclBroadcast(t.data_ptr(), t.data_ptr(), t.numel(), _DTYPES[t.dtype], src,
                                                    self.comm, self._stream(stream)))
        return t

    def send(self, t: torch.Tensor, dst: int, stream=None) -> None:
        self.nccl.check(self.nccl.lib.ncclSend(t.data_ptr(), t.numel(), _DTYPES[t.dtype], dst, self.comm,
                                               self._stream(stream)))

    def recv(self, t: torch.Tensor, src: int, stream=None) -> None:
        self.nccl.check(self.nccl.lib.ncclRecv(t.data_ptr(), t.numel(), _DTYPES[t.dtype], src, self.comm,
                                               self._stream(stream)))

    def destroy(self) -> None:
        if self.comm:
            self.nccl.lib.ncclCommDestroy(self.comm)
            self.comm = ncclComm_t()
