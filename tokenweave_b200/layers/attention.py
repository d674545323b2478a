"""Attention layer: RoPE + paged KV-cache write + causal varlen attention, with the metadata that
makes each token split a valid variable-length batch.

Counterparts: vllm/attention/layer.py:169-240 (layer), vllm/v1/attention/backends/flash_attn.py:121-137
and :674-695 (split metadata and per-split dispatch). Queries are routed by run length: runs of at
least ``PREFILL_MIN_Q`` tokens go to the tcgen05 tile kernel in 128-query tiles, shorter runs (decode
tokens, tails of chunked prompts) to the split-KV single-query kernel, one entry per token.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch
from torch import nn

from .. import ops
from ..ops import reference

PREFILL_MIN_Q = 16
_I32_FIELDS = ("positions", "slot_mapping", "cu_q", "kv_lens", "tile_seq", "tile_q0", "tok_row", "tok_seq",
               "tok_kvlen")


@dataclass
class AttentionMetadata:
    """One variable-length batch: ``B`` sequences laid out back to back in the token rows."""
    num_actual_tokens: int
    num_seqs: int
    positions: torch.Tensor          # [T] int32 absolute position of every token
    slot_mapping: torch.Tensor       # [T] int32 cache slot (block * page + offset), -1 = do not write
    cu_q: torch.Tensor               # [B+1] int32
    kv_lens: torch.Tensor            # [B] int32 keys visible to the last query of each sequence
    block_table: torch.Tensor        # [B, max_blocks] int32
    tile_seq: torch.Tensor           # prefill tiles
    tile_q0: torch.Tensor
    num_tiles: int
    tok_row: torch.Tensor            # single-query tokens
    tok_seq: torch.Tensor
    tok_kvlen: torch.Tensor
    num_single: int
    max_kv_len: int
    cu_q_cpu: list = field(default_factory=list)
    kv_lens_cpu: list = field(default_factory=list)


def plan_attention(q_lens: Sequence[int], kv_lens: Sequence[int]):
    """Host-side routing: 128-query tiles (longest causal span first) and single-query tokens."""
    if q_lens and max(q_lens) == 1 and min(q_lens) == 1:
        # a decode-only step (the common case while serving): one single-query token per sequence, no loop
        rows = np.arange(len(q_lens), dtype=np.int32)
        return [], [], rows, rows, np.asarray(kv_lens, dtype=np.int32)
    tile_seq, tile_q0, tok_row, tok_seq, tok_kv = [], [], [], [], []
    row = 0
    for b, (ql, kv) in enumerate(zip(q_lens, kv_lens)):
        if ql >= PREFILL_MIN_Q:
            for q0 in range(0, ql, 128):
                tile_seq.append(b)
                tile_q0.append(q0)
        else:
            for i in range(ql):
                tok_row.append(row + i)
                tok_seq.append(b)
                tok_kv.append(kv - ql + i + 1)
        row += ql
    if tile_seq:
        span = [kv_lens[b] - q_lens[b] + q0 for b, q0 in zip(tile_seq, tile_q0)]
        order = np.argsort(-np.asarray(span), kind="stable")
        tile_seq = [tile_seq[i] for i in order]
        tile_q0 = [tile_q0[i] for i in order]
    return tile_seq, tile_q0, tok_row, tok_seq, tok_kv


def build_attention_metadata(q_lens: Sequence[int], kv_lens: Sequence[int], positions: np.ndarray,
                             slot_mapping: np.ndarray, block_table: np.ndarray, device: torch.device,
                             pinned: Optional[torch.Tensor] = None,
                             device_buffer: Optional[torch.Tensor] = None) -> AttentionMetadata:
    """Pack every int32 array into one staging buffer, copy it to the device once, slice views."""
    q_lens = [int(x) for x in q_lens]
    kv_lens = [int(x) for x in kv_lens]
    B = len(q_lens)
    cu = np.zeros(B + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu[1:])
    tile_seq, tile_q0, tok_row, tok_seq, tok_kv = plan_attention(q_lens, kv_lens)
    arrays = {
        "positions": np.asarray(positions, dtype=np.int32), "slot_mapping": np.asarray(slot_mapping, dtype=np.int32),
        "cu_q": cu, "kv_lens": np.asarray(kv_lens, dtype=np.int32),
        "tile_seq": np.asarray(tile_seq, dtype=np.int32), "tile_q0": np.asarray(tile_q0, dtype=np.int32),
        "tok_row": np.asarray(tok_row, dtype=np.int32), "tok_seq": np.asarray(tok_seq, dtype=np.int32),
        "tok_kvlen": np.asarray(tok_kv, dtype=np.int32),
    }
    bt = np.ascontiguousarray(block_table, dtype=np.int32).reshape(B, -1)
    sizes = [(k, (arrays[k].size + 3) // 4 * 4) for k in _I32_FIELDS] + [("block_table", (bt.size + 3) // 4 * 4)]
    total = sum(s for _, s in sizes)
    if pinned is not None and pinned.numel() >= total:
        host = pinned[:total]
    else:
        host = torch.empty(total, dtype=torch.int32, pin_memory=(device.type == "cuda"))
    hv = host.numpy()
    off = 0
    offsets = {}
    for k, s in sizes:
        src = bt.reshape(-1) if k == "block_table" else arrays[k]
        hv[off:off + src.size] = src
        offsets[k] = (off, src.size)
        off += s
    if device.type != "cuda":
        dev = host
    elif device_buffer is not None and device_buffer.numel() >= total:
        # persistent device memory: the views keep their addresses from step to step, which is what a
        # captured CUDA graph needs (the layout depends only on the array sizes)
        dev = device_buffer[:total]
        dev.copy_(host, non_blocking=True)
    else:
        dev = host.to(device, non_blocking=True)
    view = {k: dev[o:o + n] for k, (o, n) in offsets.items()}
    return AttentionMetadata(
        num_actual_tokens=int(cu[-1]), num_seqs=B, positions=view["positions"], slot_mapping=view["slot_mapping"],
        cu_q=view["cu_q"], kv_lens=view["kv_lens"], block_table=view["block_table"].view(B, -1) if B else view["block_table"].view(0, 1),
        tile_seq=view["tile_seq"], tile_q0=view["tile_q0"], num_tiles=len(tile_seq), tok_row=view["tok_row"],
        tok_seq=view["tok_seq"], tok_kvlen=view["tok_kvlen"], num_single=len(tok_row),
        max_kv_len=max(kv_lens) if kv_lens else 0, cu_q_cpu=cu.tolist(), kv_lens_cpu=kv_lens)


class Attention(nn.Module):
    """Owns the layer's KV cache and runs rope -> cache write -> attention on packed qkv rows."""

    def __init__(self, num_q_heads: int, num_kv_heads: int, head_dim: int, scale: Optional[float] = None,
                 sliding_window: int = 0, logit_softcap: float = 0.0):
        super().__init__()
        self.hq, self.hkv, self.head_dim = num_q_heads, num_kv_heads, head_dim
        self.scale = scale if scale is not None else head_dim ** -0.5
        # options of the reference's attention backend (vllm/v1/attention/backends/flash_attn.py:517-538): a query
        # sees the last `sliding_window` keys only (0: all); scores pass through cap * tanh(s / cap) (0: off)
        self.window, self.softcap = int(sliding_window or 0), float(logit_softcap or 0.0)
        self.k_cache: Optional[torch.Tensor] = None   # [blocks, page, hkv, D]
        self.v_cache: Optional[torch.Tensor] = None
        self.qk_norm: Optional[tuple] = None          # (q weight [D], k weight [D], eps): per-head RMSNorm before rope

    def bind_kv_cache(self, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
        self.k_cache, self.v_cache = k_cache, v_cache

    def forward(self, qkv: torch.Tensor, cos_sin: torch.Tensor, meta: AttentionMetadata,
                out: torch.Tensor, max_ctas: int = 0) -> torch.Tensor:
        """``max_ctas``: SM budget of the prefill kernel (0: all), so that a collective running on the
        second stream keeps its SMs during attention as it does during the GEMMs."""
        n = meta.num_actual_tokens
        if n == 0:
            return out
        ops.rope_kv_write_(qkv, meta.positions, meta.slot_mapping, cos_sin, self.k_cache, self.v_cache, self.hq,
                           self.hkv, self.head_dim, qk_norm=self.qk_norm)
        q = qkv[:, : self.hq * self.head_dim]
        if not qkv.is_cuda:
            out[:n] = reference.paged_attention(q[:n], self.k_cache, self.v_cache, meta.cu_q_cpu, meta.kv_lens_cpu,
                                                meta.block_table, self.hq, self.hkv, self.head_dim, self.scale,
                                                window=self.window, softcap=self.softcap)
            return out
        ops.attn_prefill(q, self.k_cache, self.v_cache, out, meta.cu_q, meta.kv_lens, meta.block_table,
                         meta.tile_seq, meta.tile_q0, meta.num_tiles, self.hq, self.hkv, self.head_dim, self.scale,
                         max_ctas=max_ctas, window=self.window, softcap=self.softcap)
        ops.attn_decode(q, self.k_cache, self.v_cache, out, meta.tok_row, meta.tok_seq, meta.tok_kvlen,
                        meta.num_single, meta.block_table, self.hq, self.hkv, self.head_dim, self.scale,
                        meta.max_kv_len, window=self.window, softcap=self.softcap)
        return out
