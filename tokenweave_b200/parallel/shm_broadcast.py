"""One-writer / many-reader message queue over a shared-memory ring buffer: the control plane
between the engine core and its worker processes.

Counterpart of vllm/distributed/device_communicators/shm_broadcast.py:46-557. A ring of ``num_chunks``
chunks; each chunk has a header of ``1 + n_readers`` flag bytes (written, read-by-reader-i). The writer
reuses a chunk once every reader has consumed it; readers consume in order. Payloads are pickled;
a payload larger than a chunk travels in several chunks (a continuation bit in the length word).
All waits take a timeout and raise ``TimeoutError`` instead of blocking forever, and poll a
``should_stop`` callable so that a dead peer ends the wait early.
"""
from __future__ import annotations

import pickle
import struct
import time
from multiprocessing import shared_memory
from typing import Any, Callable, Optional

_LEN = struct.Struct("<Q")
_MORE = 1 << 63


class ShmRingBuffer:
    def __init__(self, n_readers: int, chunk_bytes: int = 1 << 20, num_chunks: int = 8, name: Optional[str] = None):
        self.n_readers = n_readers
        self.chunk_bytes = chunk_bytes
        self.num_chunks = num_chunks
        self.header = 1 + n_readers
        self.stride = self.header + _LEN.size + chunk_bytes
        size = self.stride * num_chunks
        if name is None:
            self.shm = shared_memory.SharedMemory(create=True, size=size)
            self.shm.buf[:size] = bytes(size)
            self.owner = True
        else:
            self.shm = shared_memory.SharedMemory(name=name)
            self.owner = False
        self.name = self.shm.name

    def handle(self) -> tuple:
        return (self.n_readers, self.chunk_bytes, self.num_chunks, self.name)

    @staticmethod
    def attach(handle: tuple) -> "ShmRingBuffer":
        n, cb, nc, name = handle
        return ShmRingBuffer(n, cb, nc, name)

    def close(self) -> None:
        try:
            self.shm.close()
            if self.owner:
                self.shm.unlink()
        except Exception:
            pass


class MessageQueue:
    """``MessageQueue.create(n_readers)`` in the writer; ``MessageQueue.attach(handle, reader_rank)`` in a reader."""

    def __init__(self, ring: ShmRingBuffer, reader_rank: Optional[int]):
        self.ring = ring
        self.reader_rank = reader_rank
        self.pos = 0

    @classmethod
    def create(cls, n_readers: int, chunk_bytes: int = 1 << 20, num_chunks: int = 8) -> "MessageQueue":
        return cls(ShmRingBuffer(n_readers, chunk_bytes, num_chunks), None)

    @classmethod
    def attach(cls, handle: tuple, reader_rank: int) -> "MessageQueue":
        return cls(ShmRingBuffer.attach(handle), reader_rank)

    def handle(self) -> tuple:
        return self.ring.handle()

    def _wait(self, ready: Callable[[], bool], timeout: Optional[float], should_stop) -> None:
        t0 = time.monotonic()
        spins = 0
        while not ready():
            spins += 1
            if spins > 200:
                time.sleep(0.0002 if spins < 5000 else 0.002)
            if should_stop is not None and spins % 64 == 0 and should_stop():
                raise ConnectionError("peer is gone")
            if timeout is not None and time.monotonic() - t0 > timeout:
                raise TimeoutError("message queue wait timed out")

    # ---- writer ----
    def enqueue(self, obj: Any, timeout: Optional[float] = None, should_stop=None) -> None:
        data = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        r = self.ring
        view = r.shm.buf
        off = 0
        while True:
            part = data[off:off + r.chunk_bytes]
            off += len(part)
            more = off < len(data)
            base = (self.pos % r.num_chunks) * r.stride

            def free() -> bool:
                return view[base] == 0 or all(view[base + 1 + i] == 1 for i in range(r.n_readers))

            self._wait(free, timeout, should_stop)
            view[base] = 0
            for i in range(r.n_readers):
                view[base + 1 + i] = 0
            _LEN.pack_into(view, base + r.header, len(part) | (_MORE if more else 0))
            view[base + r.header + _LEN.size: base + r.header + _LEN.size + len(part)] = part
            view[base] = 1          # publish last
            self.pos += 1
            if not more:
                return

    # ---- reader ----
    def dequeue(self, timeout: Optional[float] = None, should_stop=None) -> Any:
        r = self.ring
        view = r.shm.buf
        me = self.reader_rank
        parts = []
        while True:
            base = (self.pos % r.num_chunks) * r.stride
            self._wait(lambda: view[base] == 1 and view[base + 1 + me] == 0, timeout, should_stop)
            (word,) = _LEN.unpack_from(view, base + r.header)
            n = word & ~_MORE
            parts.append(bytes(view[base + r.header + _LEN.size: base + r.header + _LEN.size + n]))
            view[base + 1 + me] = 1
            self.pos += 1
            if not (word & _MORE):
                break
        return pickle.loads(b"".join(parts))

    def close(self) -> None:
        self.ring.close()
