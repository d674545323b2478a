"""A process group for control messages that lives entirely on a TCP key-value store.

Counterpart of ``StatelessProcessGroup`` (vllm/distributed/utils.py:118-250): several such groups can exist
side by side and none of them touches ``torch.distributed``'s global state, which is what a process needs
when it talks to peers outside its tensor-parallel job — data-parallel replicas agreeing on a shutdown, a
launcher handing out NCCL unique ids, tests that stand in for other nodes. Objects are pickled; every message
has its own key (``<kind>/<src>/<dst or *>/<sequence>``), consumed keys are deleted by their last reader, and
all waits have a timeout that raises ``TimeoutError`` instead of blocking for ever. Only for metadata: tensors
travel over NCCL or the shared-memory queue.
"""
from __future__ import annotations

import datetime
import pickle
import time
from typing import Any, Optional

import torch.distributed as dist


class StoreGroup:
    def __init__(self, store, rank: int, world_size: int, timeout_s: float = 300.0, host_rank: Optional[int] = 0):
        """``host_rank``: the rank whose process serves the store (None: some process outside the group). It leaves
        a barrier last, so that a barrier at the end of a job is not cut short by the store going away."""
        self.store, self.rank, self.world_size, self.timeout_s = store, rank, world_size, timeout_s
        self.host_rank = host_rank
        self._send_seq: dict[int, int] = {}
        self._recv_seq: dict[int, int] = {}
        self._bcast_seq: dict[int, int] = {}
        self._barrier_seq = 0

    @classmethod
    def create(cls, host: str, port: int, rank: int, world_size: int, timeout_s: float = 300.0) -> "StoreGroup":
        """Rank 0 hosts the store; the call returns once the store is reachable (not once all ranks joined)."""
        store = dist.TCPStore(host, port, world_size, is_master=(rank == 0),
                              timeout=datetime.timedelta(seconds=timeout_s), wait_for_workers=False)
        return cls(store, rank, world_size, timeout_s)

    # ---- plumbing ---------------------------------------------------------------------------------
    def _get(self, key: str, timeout_s: Optional[float]) -> bytes:
        deadline = time.monotonic() + (self.timeout_s if timeout_s is None else timeout_s)
        while True:
            if self.store.check([key]):
                return self.store.get(key)
            if time.monotonic() > deadline:
                raise TimeoutError(f"rank {self.rank}: no message under {key!r}")
            time.sleep(0.002)

    # ---- point to point ---------------------------------------------------------------------------
    def send_obj(self, obj: Any, dst: int) -> None:
        seq = self._send_seq.get(dst, 0)
        self._send_seq[dst] = seq + 1
        self.store.set(f"p2p/{self.rank}/{dst}/{seq}", pickle.dumps(obj))

    def recv_obj(self, src: int, timeout_s: Optional[float] = None) -> Any:
        seq = self._recv_seq.get(src, 0)
        key = f"p2p/{src}/{self.rank}/{seq}"
        data = self._get(key, timeout_s)
        self._recv_seq[src] = seq + 1
        self.store.delete_key(key)
        return pickle.loads(data)

    # ---- collectives ------------------------------------------------------------------------------
    def broadcast_obj(self, obj: Any, src: int, timeout_s: Optional[float] = None) -> Any:
        seq = self._bcast_seq.get(src, 0)
        self._bcast_seq[src] = seq + 1
        key = f"bcast/{src}/{seq}"
        if self.rank == src:
            self.store.set(key, pickle.dumps(obj))
            out = obj
        else:
            out = pickle.loads(self._get(key, timeout_s))
        # the last reader removes the message
        if self.store.add(key + "/readers", 1) == self.world_size:
            self.store.delete_key(key)
            self.store.delete_key(key + "/readers")
        return out

    def all_gather_obj(self, obj: Any, timeout_s: Optional[float] = None) -> list:
        return [self.broadcast_obj(obj if r == self.rank else None, r, timeout_s) for r in range(self.world_size)]

    def barrier(self, timeout_s: Optional[float] = None) -> None:
        """All ranks arrive, then all leave; a rank that never comes makes the others raise TimeoutError."""
        seq = self._barrier_seq
        self._barrier_seq += 1
        key = f"barrier/{seq}"
        self.store.add(key, 1)
        deadline = time.monotonic() + (self.timeout_s if timeout_s is None else timeout_s)
        while int(self.store.add(key, 0)) < self.world_size:
            if time.monotonic() > deadline:
                raise TimeoutError(f"rank {self.rank}: barrier {seq} incomplete "
                                   f"({int(self.store.add(key, 0))} of {self.world_size} ranks)")
            time.sleep(0.002)
        left = self.store.add(key + "/left", 1)
        if self.host_rank is None:
            cleanup = left == self.world_size           # whoever leaves last
        elif self.rank == self.host_rank:
            # the host leaves last and is the only one to delete the counters (a peer deleting them while the
            # host still polls would make the poll re-create them at zero)
            while left < self.world_size and time.monotonic() <= deadline:
                time.sleep(0.002)
                left = int(self.store.add(key + "/left", 0))
            cleanup = left == self.world_size
        else:
            cleanup = False
        if cleanup:
            self.store.delete_key(key)
            self.store.delete_key(key + "/left")
