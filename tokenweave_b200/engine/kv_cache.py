"""Paged KV-cache bookkeeping: a ref-counted block pool with an LRU free queue, optional
prefix-cache hashing, and the per-request slot allocator.

Counterpart of vllm/v1/core/kv_cache_manager.py:105-324 and block_pool.py. Pure CPU. The default
page is 128 tokens (one TMA box per page and 64-column half in the attention kernel) instead of the
reference's 16; any power of two from 8 to 128 works.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from typing import Optional

from .request import Request


class BlockPool:
    def __init__(self, num_blocks: int, enable_caching: bool = False):
        if num_blocks < 2:
            raise ValueError("the KV cache needs at least 2 blocks")
        self.num_blocks = num_blocks
        self.enable_caching = enable_caching
        self.ref = [0] * num_blocks
        # block 0 is reserved: out-of-range page-table entries point at it
        self.free: "OrderedDict[int, None]" = OrderedDict((i, None) for i in range(1, num_blocks))
        self.hash_of: dict[int, bytes] = {}
        self.block_of: dict[bytes, int] = {}

    @property
    def num_free(self) -> int:
        return len(self.free)

    def usage(self) -> float:
        return 1.0 - self.num_free / max(1, self.num_blocks - 1)

    def allocate(self, n: int) -> list[int]:
        if n > len(self.free):
            raise RuntimeError("out of KV blocks")
        out = []
        for _ in range(n):
            b, _ = self.free.popitem(last=False)
            h = self.hash_of.pop(b, None)
            if h is not None and self.block_of.get(h) == b:
                del self.block_of[h]
            self.ref[b] = 1
            out.append(b)
        return out

    def touch(self, b: int) -> None:
        """Take a reference on a cached block (removing it from the free queue if it was evictable)."""
        if self.ref[b] == 0:
            self.free.pop(b, None)
        self.ref[b] += 1

    def release(self, blocks: list[int]) -> None:
        # freed in reverse so that the tail of a sequence is evicted before its head
        for b in reversed(blocks):
            self.ref[b] -= 1
            if self.ref[b] == 0:
                self.free[b] = None

    def cache_block(self, b: int, h: bytes) -> None:
        if self.enable_caching and h not in self.block_of:
            self.block_of[h] = b
            self.hash_of[b] = h

    def lookup(self, h: bytes) -> Optional[int]:
        return self.block_of.get(h) if self.enable_caching else None

    def reset_prefix_cache(self) -> bool:
        """Forget every cached prefix (the KV contents are gone, e.g. after sleep). Only legal while no
        request holds blocks; returns False otherwise (vllm/v1/core/block_pool.py ``reset_prefix_cache``)."""
        if any(r > 0 for r in self.ref[1:]):
            return False
        self.hash_of.clear()
        self.block_of.clear()
        return True


def block_hashes(token_ids: list[int], block_size: int, salt: bytes = b"") -> list[bytes]:
    """Chained hash of every full block of a token sequence. ``salt`` separates sequences whose KV differs
    for the same tokens (requests served through different LoRA adapters)."""
    out = []
    prev = salt
    for i in range(0, len(token_ids) - block_size + 1, block_size):
        m = hashlib.sha256(prev)
        m.update(b",".join(str(t).encode() for t in token_ids[i:i + block_size]))
        prev = m.digest()
        out.append(prev)
    return out


class KVCacheManager:
    def __init__(self, num_blocks: int, block_size: int, enable_caching: bool = False):
        self.block_size = block_size
        self.pool = BlockPool(num_blocks, enable_caching)
        self.enable_caching = enable_caching
        self.prefix_queries = 0        # blocks looked up / found in the prefix cache since start
        self.prefix_hits = 0
        self.track_published = False   # a KV connector wants to know which blocks became full
        self.newly_published: list[tuple[int, bytes]] = []     # (block id, hash) since the engine last took them

    def get_computed_blocks(self, req: Request) -> tuple[list[int], int]:
        """Longest cached prefix of the request's prompt: (block ids, number of tokens)."""
        if not self.enable_caching:
            return [], 0
        blocks = []
        # never reuse the whole prompt: the last token must be recomputed to produce logits
        usable = (req.num_tokens - 1) // self.block_size
        for h in self._hashes(req, usable):
            b = self.pool.lookup(h)
            if b is None:
                break
            blocks.append(b)
        self.prefix_queries += usable
        self.prefix_hits += len(blocks)
        return blocks, len(blocks) * self.block_size

    def allocate_slots(self, req: Request, num_new_tokens: int, cached_blocks: Optional[list[int]] = None) -> bool:
        """Make sure ``req`` owns enough blocks for ``num_computed_tokens + num_new_tokens`` tokens.
        Returns False (and changes nothing) if the pool cannot provide them."""
        if not cached_blocks and (req.num_computed_tokens + num_new_tokens) <= len(req.block_ids) * self.block_size:
            return True                    # the common decode step: the last block still has room
        cached_blocks = cached_blocks or []
        have = len(req.block_ids) + len(cached_blocks)
        need_total = (req.num_computed_tokens + len(cached_blocks) * 0 + num_new_tokens + self.block_size - 1) // self.block_size
        need = max(0, need_total - have)
        evictable_cached = sum(1 for b in cached_blocks if self.pool.ref[b] == 0)
        if need > self.pool.num_free - evictable_cached:
            return False
        for b in cached_blocks:
            self.pool.touch(b)
        req.block_ids.extend(cached_blocks)
        req.block_ids.extend(self.pool.allocate(need))
        return True

    def _hashes(self, req: Request, num_blocks: int) -> list[bytes]:
        """Chained hashes of the request's first ``num_blocks`` full blocks. The chain is kept on the request
        and only extended: tokens are append-only, so a block's hash never changes once it is full."""
        chain = req.block_hash_chain
        bs = self.block_size
        if len(chain) < num_blocks:
            prev = chain[-1] if chain else req.cache_salt
            for i in range(len(chain), num_blocks):
                m = hashlib.sha256(prev)
                m.update(b",".join(str(req.token_at(j)).encode() for j in range(i * bs, (i + 1) * bs)))
                prev = m.digest()
                chain.append(prev)
        return chain[:num_blocks]

    def cache_full_blocks(self, req: Request) -> None:
        """Publish the blocks that became full since the last call (per-step cost: O(new blocks))."""
        if not self.enable_caching:
            return
        full = req.num_computed_tokens // self.block_size
        if full <= req.num_published_blocks:
            return
        hashes = self._hashes(req, full)
        for i in range(req.num_published_blocks, full):
            self.pool.cache_block(req.block_ids[i], hashes[i])
            if self.track_published:
                self.newly_published.append((req.block_ids[i], hashes[i]))
        req.num_published_blocks = full

    def prefix_hashes(self, req: Request) -> list[bytes]:
        """Hashes of the prompt blocks a request may take from a cache (never the block of its last token)."""
        return self._hashes(req, (req.num_tokens - 1) // self.block_size)

    def free(self, req: Request) -> None:
        self.pool.release(req.block_ids)
        req.block_ids = []
        req.num_published_blocks = 0       # the next owner of these block ids starts over; the hash chain stays

    def usage(self) -> float:
        return self.pool.usage()
