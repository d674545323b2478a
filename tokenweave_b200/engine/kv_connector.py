"""KV-transfer connectors: KV-cache blocks leave one engine and enter another, through shared storage
(``SharedStorageConnector``) or over the network through a key-value store that one of the engines hosts
(``TcpStoreConnector``).

Counterpart of the reference's ``vllm/distributed/kv_transfer/`` (connector interface, ``KVTransferConfig`` with
``kv_connector`` / ``kv_role`` / ``kv_connector_extra_config``, the scheduler hooks at
vllm/v1/core/sched/scheduler.py:319-367): the mechanism behind disaggregated prefill (a *producer* instance
prefills and publishes, a *consumer* instance picks the blocks up and only decodes) and behind an external
prefix cache shared by several replicas.

Blocks are identified by the prefix-cache hash chain (``engine/kv_cache.py``), so whatever one engine stored
is found by any engine that serves the same model with the same block size, adapter and tensor-parallel
layout. One file per (block, rank): the ranks of a tensor- or pipeline-parallel replica each write their own
shard of a block; a block counts as available once every rank's file is there. Files are written to a temporary
name and renamed, so a reader never sees a partial block.

``TcpStoreConnector`` is the networked form (the place of the reference's P2P / LMCache / Mooncake pipes,
vllm/distributed/kv_transfer/kv_connector/): blocks travel as byte strings (a small JSON header and the raw tensor
bytes, nothing that is unpickled) to and from a ``torch.distributed.TCPStore``; the engine whose configuration says
``"is_master": true`` hosts the store, every other engine and every worker connects to ``host:port``. A producer and
a consumer on different machines need no common file system.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Optional

import torch

ROLES = ("kv_producer", "kv_consumer", "kv_both")
CONNECTORS = ("SharedStorageConnector", "TcpStoreConnector")


@dataclass
class KVTransferConfig:
    kv_connector: str = "SharedStorageConnector"
    kv_role: str = "kv_both"
    shared_storage_path: str = ""
    host: str = "127.0.0.1"          # TcpStoreConnector: where the store listens
    port: int = 0
    is_master: bool = False          # TcpStoreConnector: this engine hosts the store
    timeout_s: float = 60.0

    @staticmethod
    def from_user(value) -> Optional["KVTransferConfig"]:
        """None, a ``KVTransferConfig``, or the reference's dict layout."""
        if value is None or isinstance(value, KVTransferConfig):
            return value
        if not isinstance(value, dict):
            raise TypeError("kv_transfer_config must be a dict")
        extra = value.get("kv_connector_extra_config") or {}
        cfg = KVTransferConfig(value.get("kv_connector", "SharedStorageConnector"), value.get("kv_role", "kv_both"),
                               extra.get("shared_storage_path", value.get("shared_storage_path", "")),
                               str(extra.get("host", "127.0.0.1")), int(extra.get("port", 0)),
                               bool(extra.get("is_master", False)), float(extra.get("timeout_s", 60.0)))
        if cfg.kv_connector not in CONNECTORS:
            raise ValueError(f"unknown kv_connector {cfg.kv_connector!r} (available: {', '.join(CONNECTORS)})")
        if cfg.kv_role not in ROLES:
            raise ValueError(f"kv_role must be one of {ROLES}")
        if cfg.kv_connector == "SharedStorageConnector" and not cfg.shared_storage_path:
            raise ValueError("SharedStorageConnector needs kv_connector_extra_config['shared_storage_path']")
        if cfg.kv_connector == "TcpStoreConnector" and cfg.port <= 0:
            raise ValueError("TcpStoreConnector needs kv_connector_extra_config['port'] (and 'host', 'is_master')")
        return cfg

    @property
    def can_save(self) -> bool:
        return self.kv_role in ("kv_producer", "kv_both")

    @property
    def can_load(self) -> bool:
        return self.kv_role in ("kv_consumer", "kv_both")


class SharedStorageConnector:
    """``rank`` / ``world`` are the global rank and size of the replica's worker group; the scheduler side uses
    rank 0 and only asks :meth:`num_matched`."""

    def __init__(self, cfg: KVTransferConfig, rank: int = 0, world: int = 1, fingerprint: str = ""):
        """``fingerprint`` names what must agree between the engines that share the directory (model, dtype,
        block size, layer count, parallel layout): it becomes a sub-directory, so two models that point at the
        same path never exchange blocks."""
        self.cfg, self.rank, self.world = cfg, rank, world
        self.root = os.path.join(cfg.shared_storage_path, fingerprint) if fingerprint else cfg.shared_storage_path
        os.makedirs(self.root, exist_ok=True)

    def _file(self, block_hash: bytes, rank: int) -> str:
        return os.path.join(self.root, f"{block_hash.hex()}.r{rank}of{self.world}.pt")

    def available(self, block_hash: bytes) -> bool:
        return all(os.path.exists(self._file(block_hash, r)) for r in range(self.world))

    def num_matched(self, hashes) -> int:
        """How many leading blocks of a hash chain the store can supply."""
        n = 0
        for h in hashes:
            if not self.available(h):
                break
            n += 1
        return n

    def save_block(self, block_hash: bytes, k: torch.Tensor, v: torch.Tensor) -> None:
        """``k`` / ``v``: this rank's ``[layers, page, kv_heads, head_dim]`` slices of one block."""
        path = self._file(block_hash, self.rank)
        if os.path.exists(path):
            return
        tmp = f"{path}.tmp{os.getpid()}"
        torch.save({"k": k.cpu().contiguous(), "v": v.cpu().contiguous()}, tmp)
        os.replace(tmp, path)

    def load_block(self, block_hash: bytes, expect_shape=None) -> tuple[torch.Tensor, torch.Tensor]:
        """Tensors only (``weights_only``): the directory is written by other processes. ``expect_shape`` is
        the ``[layers, page, kv_heads, head_dim]`` shape the caller's cache needs."""
        d = torch.load(self._file(block_hash, self.rank), map_location="cpu", weights_only=True)
        k, v = d["k"], d["v"]
        if expect_shape is not None and (tuple(k.shape) != tuple(expect_shape) or tuple(v.shape) != tuple(expect_shape)):
            raise ValueError(f"stored KV block has shape {tuple(k.shape)}, this engine needs {tuple(expect_shape)}")
        return k, v


_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32,
           "float8_e4m3fn": torch.float8_e4m3fn, "int8": torch.int8}


def encode_block(k: torch.Tensor, v: torch.Tensor) -> bytes:
    """``k`` and ``v`` of one block as bytes: 4-byte header length, a JSON header (dtype, shape), the raw bytes."""
    k, v = k.detach().cpu().contiguous(), v.detach().cpu().contiguous()
    name = str(k.dtype).replace("torch.", "")
    if name not in _DTYPES or v.dtype != k.dtype or v.shape != k.shape:
        raise ValueError(f"cannot encode KV blocks of dtype {k.dtype} / shapes {tuple(k.shape)}, {tuple(v.shape)}")
    head = json.dumps({"dtype": name, "shape": list(k.shape)}).encode()
    raw = lambda t: t.view(torch.uint8).numpy().tobytes()          # noqa: E731
    return struct.pack("<I", len(head)) + head + raw(k) + raw(v)


def decode_block(data: bytes) -> tuple[torch.Tensor, torch.Tensor]:
    (n,) = struct.unpack_from("<I", data, 0)
    head = json.loads(data[4:4 + n].decode())
    dtype, shape = _DTYPES[head["dtype"]], tuple(int(x) for x in head["shape"])
    count = 1
    for x in shape:
        count *= x
    nbytes = count * torch.empty((), dtype=dtype).element_size()
    body = memoryview(data)[4 + n:]
    if len(body) != 2 * nbytes:
        raise ValueError(f"KV block of {len(body)} bytes does not hold two tensors of shape {shape}")
    one = lambda b: torch.frombuffer(bytearray(b), dtype=torch.uint8).view(dtype).reshape(shape)     # noqa: E731
    return one(body[:nbytes]), one(body[nbytes:])


class TcpStoreConnector:
    """Same interface as :class:`SharedStorageConnector`; the blocks live in a ``TCPStore``. ``host_store``: this
    instance may host the store (the engine-side instance of the configuration with ``is_master``); worker-side
    instances always connect as clients."""

    def __init__(self, cfg: KVTransferConfig, rank: int = 0, world: int = 1, fingerprint: str = "",
                 host_store: bool = False):
        from datetime import timedelta

        from torch.distributed import TCPStore
        self.cfg, self.rank, self.world, self.prefix = cfg, rank, world, fingerprint
        key = (cfg.host, cfg.port)
        hosted = _HOSTED_STORES.get(key)
        if hosted is not None:
            self.store = hosted                      # the engine of this process hosts it: use it directly
        else:
            self.store = TCPStore(cfg.host, cfg.port, is_master=bool(host_store and cfg.is_master),
                                  wait_for_workers=False, timeout=timedelta(seconds=cfg.timeout_s))
            if host_store and cfg.is_master:
                _HOSTED_STORES[key] = self.store

    def _key(self, block_hash: bytes, rank: int) -> str:
        return f"{self.prefix}/{block_hash.hex()}.r{rank}of{self.world}"

    def available(self, block_hash: bytes) -> bool:
        return bool(self.store.check([self._key(block_hash, r) for r in range(self.world)]))

    def num_matched(self, hashes) -> int:
        n = 0
        for h in hashes:
            if not self.available(h):
                break
            n += 1
        return n

    def save_block(self, block_hash: bytes, k: torch.Tensor, v: torch.Tensor) -> None:
        key = self._key(block_hash, self.rank)
        if not self.store.check([key]):
            self.store.set(key, encode_block(k, v))

    def load_block(self, block_hash: bytes, expect_shape=None) -> tuple[torch.Tensor, torch.Tensor]:
        k, v = decode_block(self.store.get(self._key(block_hash, self.rank)))
        if expect_shape is not None and (tuple(k.shape) != tuple(expect_shape) or tuple(v.shape) != tuple(expect_shape)):
            raise ValueError(f"stored KV block has shape {tuple(k.shape)}, this engine needs {tuple(expect_shape)}")
        return k, v


_HOSTED_STORES: dict = {}      # (host, port) -> the TCPStore this process hosts


def make_connector(cfg: KVTransferConfig, rank: int, world: int, fingerprint: str, host_store: bool = False):
    """The connector a configuration names. ``host_store``: the caller is the engine side (it may host a store)."""
    if cfg.kv_connector == "TcpStoreConnector":
        return TcpStoreConnector(cfg, rank, world, fingerprint, host_store)
    return SharedStorageConnector(cfg, rank, world, fingerprint)


def kv_fingerprint(config) -> str:
    """Identity of a KV layout: engines whose fingerprints differ keep their blocks apart."""
    import hashlib
    m, par = config.model, config.parallel
    key = (m.name, m.architecture, m.num_layers, m.hidden_size, m.num_kv_heads, m.head_dim, str(m.dtype),
           config.cache.block_size, par.tensor_parallel_size, getattr(par, "pipeline_parallel_size", 1))
    return hashlib.sha256(repr(key).encode()).hexdigest()[:16]
