"""KV-transfer connector: KV-cache blocks leave one engine and enter another through shared storage.

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
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

ROLES = ("kv_producer", "kv_consumer", "kv_both")


@dataclass
class KVTransferConfig:
    kv_connector: str = "SharedStorageConnector"
    kv_role: str = "kv_both"
    shared_storage_path: str = ""

    @staticmethod
    def from_user(value) -> Optional["KVTransferConfig"]:
        """None, a ``KVTransferConfig``, or the reference's dict layout."""
        if value is None or isinstance(value, KVTransferConfig):
            return value
        if not isinstance(value, dict):
            raise TypeError("kv_transfer_config must be a dict")
        extra = value.get("kv_connector_extra_config") or {}
        cfg = KVTransferConfig(value.get("kv_connector", "SharedStorageConnector"), value.get("kv_role", "kv_both"),
                               extra.get("shared_storage_path", value.get("shared_storage_path", "")))
        if cfg.kv_connector != "SharedStorageConnector":
            raise ValueError(f"unknown kv_connector {cfg.kv_connector!r} (available: SharedStorageConnector)")
        if cfg.kv_role not in ROLES:
            raise ValueError(f"kv_role must be one of {ROLES}")
        if not cfg.shared_storage_path:
            raise ValueError("SharedStorageConnector needs kv_connector_extra_config['shared_storage_path']")
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


def kv_fingerprint(config) -> str:
    """Identity of a KV layout: engines whose fingerprints differ keep their blocks apart."""
    import hashlib
    m, par = config.model, config.parallel
    key = (m.name, m.architecture, m.num_layers, m.hidden_size, m.num_kv_heads, m.head_dim, str(m.dtype),
           config.cache.block_size, par.tensor_parallel_size, getattr(par, "pipeline_parallel_size", 1))
    return hashlib.sha256(repr(key).encode()).hexdigest()[:16]
