"""Operator layer: one Python function per hot op.

CUDA tensors go to the hand-written sm_100a kernels in ``_C.so`` (through :mod:`._native`; a missing
library raises). CPU tensors go to the PyTorch references in :mod:`.reference`, which are also the
oracle the kernels are tested against.

Reference counterpart of this layer: vllm/_custom_ops.py:184-221 and csrc/torch_bindings.cpp:146-196.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _native, gemm_table, reference

__all__ = [
    "gemm", "rmsnorm", "rmsnorm_copy_", "add_rmsnorm_", "rope_kv_write_", "swiglu", "embedding", "argmax",
    "quant_fp8", "rmsnorm_quant_fp8", "quant_int8", "rmsnorm_quant_int8", "gather_cache", "convert_fp8", "permute_cols",
    "gemm_fp8", "activation", "copy_pages", "swap_pages", "merge_attn_states", "attn_prefill", "attn_decode", "moe_router", "moe_align", "moe_scatter", "moe_combine", "status_word",
    "check_status", "reset_status", "STATUS_CODES", "KernelStatusError",
]

STATUS_CODES = {1: "mbarrier wait timed out", 2: "peer signal wait timed out", 4: "bad argument",
                8: "tile-ready flag wait timed out"}


class KernelStatusError(RuntimeError):
    """A kernel gave up on a bounded wait (or failed a device-side check) and said so."""

    def __init__(self, code: int):
        self.code = code
        what = ", ".join(v for k, v in STATUS_CODES.items() if code & k) or "unknown"
        super().__init__(f"device status word = {code:#x}: {what}")


_status: dict[int, torch.Tensor] = {}


def status_word(device=None) -> torch.Tensor:
    """The int32 word kernels OR their error codes into (one per device, zero when healthy)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device=None) -> None:
    """Synchronising read of the status word; raises :class:`KernelStatusError` if it is non-zero."""
    code = int(status_word(device).item())
    if code != 0:
        raise KernelStatusError(code)


def reset_status(device=None) -> None:
    status_word(device).zero_()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check_bf16(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and t.dtype != torch.bfloat16:
            raise TypeError(f"the sm_100a kernels take bfloat16 tensors, got {t.dtype}")


def _row_stride(t: torch.Tensor) -> int:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("expected a 2-D tensor with contiguous rows")
    return t.stride(0)


# ---------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, *,
         bias: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None, swiglu: bool = False,
         max_ctas: int = 0, tile_expert: Optional[torch.Tensor] = None,
         num_m_tiles: Optional[torch.Tensor] = None, n_per_expert: int = 0, tile_rows: int = 128) -> torch.Tensor:
    """``out = a @ w.T`` (+bias, *row_scale); with ``swiglu`` the weight is ``[gate; up]`` and the
    output is ``silu(a@gate.T) * (a@up.T)``. Grouped mode (``tile_expert`` given): every ``tile_rows``-row
    tile of ``a`` multiplies the weight block of its expert, ``w`` being ``[E * n_per_expert, K]``;
    ``tile_rows`` is 128 (single-CTA tiles) or 256 (experts padded to 256 rows: the groups run on CTA pairs)."""
    M, K = a.shape
    rows_b = w.shape[0]
    per_expert = n_per_expert if tile_expert is not None else rows_b
    N = per_expert // 2 if swiglu else per_expert
    if out is None:
        out = torch.empty(M, N, dtype=a.dtype, device=a.device)
    if not a.is_cuda:
        if tile_expert is not None:
            raise NotImplementedError("grouped GEMM on CPU goes through reference.moe_experts")
        res = reference.gemm_swiglu(a, w, row_scale) if swiglu else reference.gemm(a, w, bias, row_scale)
        out.copy_(res)
        return out
    _check_bf16(a, w, out, bias)
    if tile_expert is not None and tile_rows == 256:
        if bias is not None:
            raise ValueError("the grouped GEMM has no bias")
        _native.call("tw_gemm_bf16_grouped256", a.data_ptr(), _row_stride(a), w.data_ptr(), _row_stride(w), rows_b,
                     out.data_ptr(), _row_stride(out), _p(row_scale), M, N, K, int(swiglu),
                     per_expert // 2 if swiglu else 0, _p(tile_expert), _p(num_m_tiles), per_expert, max_ctas,
                     status_word(a.device).data_ptr(), _stream(),
                     tag=f"[grouped {M}x{N}x{K}{'+swiglu' if swiglu else ''}]" if _native._timing is not None else "")
        return out
    _native.call("tw_gemm_bf16", a.data_ptr(), _row_stride(a), w.data_ptr(), _row_stride(w), rows_b,
                 out.data_ptr(), _row_stride(out), _p(bias), _p(row_scale), M, N, K, int(swiglu),
                 per_expert // 2 if swiglu else 0, _p(tile_expert), _p(num_m_tiles), per_expert, max_ctas,
                 0 if tile_expert is not None else gemm_table.lookup(M, N, K, swiglu, max_ctas),
                 status_word(a.device).data_ptr(), _stream(),
                 tag=f"[{M}x{N}x{K}{'+swiglu' if swiglu else ''}]" if _native._timing is not None else "")
    return out


FP8 = torch.float8_e4m3fn


def quant_fp8(x: torch.Tensor, scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
              max_ctas: int = 0):
    """bf16 ``[T, H]`` -> (e4m3 ``[T, H]``, fp32 scales). ``scale`` None: dynamic per-token scales
    ``max|row| / 448`` (``[T]``); else the given one-element tensor is used for every row (static)."""
    T, H = x.shape
    if out is None:
        out = torch.empty(T, H, dtype=FP8, device=x.device)
    if not x.is_cuda:
        q, s = reference.quant_fp8(x, scale)
        out.copy_(q)
        return out, s
    _check_bf16(x)
    scales = torch.empty(T, dtype=torch.float32, device=x.device) if scale is None else scale
    _native.call("tw_quant_fp8", x.data_ptr(), _row_stride(x), out.data_ptr(), _row_stride(out), scales.data_ptr(),
                 T, H, int(scale is None), max_ctas, _stream())
    return out, scales


def rmsnorm_quant_fp8(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None,
                      scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, max_ctas: int = 0):
    """``q = e4m3(rmsnorm(x [+ residual]) * weight / scale)``; with ``residual`` the sum is written back to
    ``residual`` first. Returns ``(q, scales)`` like :func:`quant_fp8`."""
    T, H = x.shape
    if out is None:
        out = torch.empty(T, H, dtype=FP8, device=x.device)
    if not x.is_cuda:
        if residual is not None:
            residual.copy_((x + residual))
            y = reference.rmsnorm(residual, weight, eps)
        else:
            y = reference.rmsnorm(x, weight, eps)
        q, s = reference.quant_fp8(y, scale)
        out.copy_(q)
        return out, s
    _check_bf16(x, weight, residual)
    scales = torch.empty(T, dtype=torch.float32, device=x.device) if scale is None else scale
    _native.call("tw_rmsnorm_quant_fp8", x.data_ptr(), _p(residual), weight.data_ptr(), out.data_ptr(),
                 _row_stride(out), scales.data_ptr(), T, H, _row_stride(x),
                 _row_stride(residual) if residual is not None else 0, float(eps), int(scale is None), max_ctas,
                 _stream())
    return out, scales


def gemm_fp8(a: torch.Tensor, w: torch.Tensor, a_scale: Optional[torch.Tensor], w_scale: Optional[torch.Tensor],
             out: Optional[torch.Tensor] = None, *, bias: Optional[torch.Tensor] = None, swiglu: bool = False,
             max_ctas: int = 0, plan: int = 0) -> torch.Tensor:
    """``out[m, n] = (a @ w.T)[m, n] * a_scale[m] * w_scale[n] + bias[n]`` in bf16, ``a`` ``[M, K]`` and ``w``
    ``[N, K]`` being e4m3 (per-token and per-output-channel scales, fp32, either may be None). With
    ``swiglu`` the weight is ``[gate; up]`` and the result ``silu(gate part) * (up part)``. ``plan``: 0 = the
    library's cost model, else kernel * 1000 + tile width (1 = single-CTA tiles, 2 = CTA pairs)."""
    M, K = a.shape
    rows_b = w.shape[0]
    N = rows_b // 2 if swiglu else rows_b
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    if not a.is_cuda:
        out.copy_(reference.gemm_fp8(a, w, a_scale, w_scale, bias, swiglu))
        return out
    if a.dtype != FP8 or w.dtype != FP8:
        raise TypeError("gemm_fp8 takes float8_e4m3fn operands")
    _check_bf16(out, bias)
    for s, n in ((a_scale, M), (w_scale, rows_b)):
        if s is not None and (s.dtype != torch.float32 or s.numel() != n or not s.is_contiguous()):
            raise ValueError("scales must be contiguous fp32 vectors of one value per row / output channel")
    _native.call("tw_gemm_fp8", a.data_ptr(), _row_stride(a), w.data_ptr(), _row_stride(w), rows_b, out.data_ptr(),
                 _row_stride(out), _p(bias), _p(a_scale), _p(w_scale), M, N, K, int(swiglu), N if swiglu else 0,
                 None, None, rows_b, max_ctas, int(plan) or gemm_table.lookup(M, N, K, swiglu, max_ctas, fp8=True),
                 status_word(a.device).data_ptr(), _stream(),
                 tag=f"[fp8 {M}x{N}x{K}{'+swiglu' if swiglu else ''}]" if _native._timing is not None else "")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None,
            max_ctas: int = 0) -> torch.Tensor:
    if out is None:
        out = torch.empty_like(x)
    if not x.is_cuda:
        out.copy_(reference.rmsnorm(x, weight, eps))
        return out
    _check_bf16(x, weight, out)
    T, H = x.shape
    _native.call("tw_rmsnorm", x.data_ptr(), out.data_ptr(), weight.data_ptr(), T, H, _row_stride(x),
                 _row_stride(out), eps, max_ctas, _stream())
    return out


def rmsnorm_copy_(x: torch.Tensor, residual_out: torch.Tensor, weight: torch.Tensor, eps: float,
                  max_ctas: int = 0) -> None:
    """``residual_out = x; x = rmsnorm(x) * w`` (first-layer helper)."""
    if not x.is_cuda:
        reference.rmsnorm_copy_(x, residual_out, weight, eps)
        return
    _check_bf16(x, weight, residual_out)
    T, H = x.shape
    _native.call("tw_rmsnorm_copy", x.data_ptr(), residual_out.data_ptr(), weight.data_ptr(), T, H,
                 _row_stride(x), _row_stride(residual_out), eps, max_ctas, _stream())


def add_rmsnorm_(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                 max_ctas: int = 0) -> None:
    """``x += residual; residual = x; x = rmsnorm(x) * w`` in place."""
    if not x.is_cuda:
        reference.add_rmsnorm_(x, residual, weight, eps)
        return
    _check_bf16(x, weight, residual)
    T, H = x.shape
    _native.call("tw_add_rmsnorm", x.data_ptr(), residual.data_ptr(), weight.data_ptr(), T, H, _row_stride(x),
                 _row_stride(residual), eps, max_ctas, _stream())


def rope_kv_write_(qkv: torch.Tensor, positions: torch.Tensor, slots: Optional[torch.Tensor],
                   cos_sin: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                   hq: int, hkv: int, head_dim: int, write_k_back: bool = False,
                   qk_norm: Optional[tuple] = None) -> None:
    """Rotate q (and k) of the first ``len(positions)`` rows of ``qkv`` and write k, v to the cache.
    ``qk_norm = (q_weight, k_weight, eps)`` RMS-normalises every q and k head over ``head_dim`` first
    (the Qwen3 layout), in the same launch."""
    T = positions.shape[0]
    if T == 0:
        return
    if not qkv.is_cuda:
        reference.rope_kv_write_(qkv[:T], positions, slots, cos_sin, k_cache, v_cache, hq, hkv, head_dim,
                                 write_k_back=True, qk_norm=qk_norm)
        return
    _check_bf16(qkv, k_cache, v_cache)
    assert positions.dtype == torch.int32 and (slots is None or slots.dtype == torch.int32)
    assert cos_sin.dtype == torch.float32 and cos_sin.shape[1] == head_dim
    if qk_norm is not None:
        qw, kw, eps = qk_norm
        _check_bf16(qw, kw)
        assert qw.numel() == head_dim and kw.numel() == head_dim
        _native.call("tw_rope_kv_write_qknorm", qkv.data_ptr(), _row_stride(qkv), positions.data_ptr(), _p(slots),
                     cos_sin.data_ptr(), _p(k_cache), _p(v_cache), T, hq, hkv, head_dim, int(write_k_back),
                     qw.data_ptr(), kw.data_ptr(), float(eps), _stream())
        return
    _native.call("tw_rope_kv_write", qkv.data_ptr(), _row_stride(qkv), positions.data_ptr(), _p(slots),
                 cos_sin.data_ptr(), _p(k_cache), _p(v_cache), T, hq, hkv, head_dim, int(write_k_back),
                 _stream())


def swiglu(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, d2 = x.shape
    d = d2 // 2
    if out is None:
        out = torch.empty(T, d, dtype=x.dtype, device=x.device)
    if not x.is_cuda:
        out.copy_(reference.swiglu(x))
        return out
    _check_bf16(x, out)
    _native.call("tw_swiglu", x.data_ptr(), _row_stride(x), out.data_ptr(), _row_stride(out), T, d, _stream())
    return out


def activation(x: torch.Tensor, kind: str, out: Optional[torch.Tensor] = None, param: float = 0.0) -> torch.Tensor:
    """Gated (``*_and_mul``: ``x`` is ``[T, 2d]``) or unary (``x`` is ``[T, d]``) activation; the kinds
    are the keys of ``reference.ACTIVATION_KINDS`` (vllm/model_executor/layers/activation.py)."""
    code = reference.ACTIVATION_KINDS[kind]
    T = x.shape[0]
    d = x.shape[1] // 2 if code <= 4 else x.shape[1]
    if out is None:
        out = torch.empty(T, d, dtype=x.dtype, device=x.device)
    if not x.is_cuda:
        out.copy_(reference.activation(x, kind, param))
        return out
    _check_bf16(x, out)
    _native.call("tw_activation", x.data_ptr(), _row_stride(x), out.data_ptr(), _row_stride(out), T, d, code,
                 float(param), _stream())
    return out


def quant_int8(x: torch.Tensor, scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               max_ctas: int = 0):
    """bf16 ``[T, H]`` -> (int8 ``[T, H]``, fp32 scales), symmetric. ``scale`` None: dynamic per-token scales
    ``max|row| / 127``; else the given one-element tensor for every row (the reference's
    ``dynamic_scaled_int8_quant`` / ``static_scaled_int8_quant``)."""
    T, H = x.shape
    if out is None:
        out = torch.empty(T, H, dtype=torch.int8, device=x.device)
    if not x.is_cuda:
        q, s = reference.quant_int8(x, scale)
        out.copy_(q)
        return out, s
    _check_bf16(x)
    scales = torch.empty(T, dtype=torch.float32, device=x.device) if scale is None else scale
    _native.call("tw_quant_int8", x.data_ptr(), _row_stride(x), out.data_ptr(), _row_stride(out), scales.data_ptr(),
                 T, H, int(scale is None), max_ctas, _stream())
    return out, scales


def gemm_int8(a: torch.Tensor, w: torch.Tensor, a_scale: Optional[torch.Tensor], w_scale: Optional[torch.Tensor],
              out: Optional[torch.Tensor] = None, *, bias: Optional[torch.Tensor] = None, swiglu: bool = False,
              max_ctas: int = 0, plan: int = 0) -> torch.Tensor:
    """``out[m, n] = (a @ w.T)[m, n] * a_scale[m] * w_scale[n] + bias[n]`` in bf16 for int8 ``a`` ``[M, K]`` and
    ``w`` ``[N, K]`` (symmetric quantisation, exact 32-bit integer accumulation on the tensor cores; scales fp32,
    either may be None). With ``swiglu`` the weight is ``[gate; up]`` and the result ``silu(gate part) * (up
    part)``. ``plan``: 0 = the library's choice, else 2000 + tile width (CTA pairs)."""
    M, K = a.shape
    rows_b = w.shape[0]
    N = rows_b // 2 if swiglu else rows_b
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    if not a.is_cuda:
        out.copy_(reference.gemm_int8(a, w, a_scale, w_scale, bias, swiglu))
        return out
    if a.dtype != torch.int8 or w.dtype != torch.int8:
        raise TypeError("gemm_int8 takes int8 operands")
    _check_bf16(out, bias)
    for s, n in ((a_scale, M), (w_scale, rows_b)):
        if s is not None and (s.dtype != torch.float32 or s.numel() != n or not s.is_contiguous()):
            raise ValueError("scales must be contiguous fp32 vectors of one value per row / output channel")
    _native.call("tw_gemm_int8", a.data_ptr(), _row_stride(a), w.data_ptr(), _row_stride(w), out.data_ptr(),
                 _row_stride(out), _p(bias), _p(a_scale), _p(w_scale), M, N, K, int(swiglu), max_ctas, int(plan),
                 status_word(a.device).data_ptr(), _stream(),
                 tag=f"[int8 {M}x{N}x{K}{'+swiglu' if swiglu else ''}]" if _native._timing is not None else "")
    return out


def rmsnorm_quant_int8(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None,
                       scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, max_ctas: int = 0):
    """``q = int8(rmsnorm(x [+ residual]) * weight / scale)``; with ``residual`` the sum is written back to
    ``residual`` first. Returns ``(q, scales)`` like :func:`quant_int8`."""
    T, H = x.shape
    if out is None:
        out = torch.empty(T, H, dtype=torch.int8, device=x.device)
    if not x.is_cuda:
        if residual is not None:
            residual.copy_((x + residual))
            y = reference.rmsnorm(residual, weight, eps)
        else:
            y = reference.rmsnorm(x, weight, eps)
        q, s = reference.quant_int8(y, scale)
        out.copy_(q)
        return out, s
    _check_bf16(x, weight)
    scales = torch.empty(T, dtype=torch.float32, device=x.device) if scale is None else scale
    _native.call("tw_rmsnorm_quant_int8", x.data_ptr(), None if residual is None else residual.data_ptr(),
                 weight.data_ptr(), out.data_ptr(), _row_stride(out), scales.data_ptr(), T, H, _row_stride(x),
                 0 if residual is None else _row_stride(residual), eps, int(scale is None), max_ctas, _stream())
    return out, scales


def gather_cache(cache: torch.Tensor, block_table: torch.Tensor, cu_seq: torch.Tensor, total_rows: int,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The cache rows of every sequence (``cu_seq``: ``[batch + 1]`` int32 prefix sums of the lengths, on the
    cache's device), in block-table order, as one contiguous ``[total_rows, kv_heads, D]`` tensor."""
    page = cache.shape[1]
    if out is None:
        out = torch.empty(total_rows, *cache.shape[2:], dtype=cache.dtype, device=cache.device)
    if not cache.is_cuda:
        lens = (cu_seq[1:] - cu_seq[:-1]).tolist()
        out.copy_(reference.gather_cache(cache, block_table, lens))
        return out
    _check_bf16(cache)
    row_elems = cache[0, 0].numel()
    _native.call("tw_gather_cache", cache.data_ptr(), out.data_ptr(), block_table.data_ptr(), cu_seq.data_ptr(),
                 block_table.shape[0], block_table.shape[1], page, row_elems, _stream())
    return out


def convert_fp8(src: torch.Tensor, scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 -> e4m3 (``src / scale``) or e4m3 -> bf16 (``src * scale``), by the dtype of ``src``: how a KV cache
    is stored in / read back from fp8 (``convert_fp8`` of the reference's cache kernels)."""
    to_fp8 = src.dtype == torch.bfloat16
    if out is None:
        out = torch.empty(src.shape, dtype=FP8 if to_fp8 else torch.bfloat16, device=src.device)
    if not src.is_cuda:
        out.copy_((src.float() / scale).clamp(-448, 448).to(FP8) if to_fp8 else (src.float() * scale).to(torch.bfloat16))
        return out
    assert src.is_contiguous() and out.is_contiguous()
    _native.call("tw_convert_fp8", src.data_ptr(), out.data_ptr(), src.numel(), float(scale), int(to_fp8), _stream())
    return out


def permute_cols(x: torch.Tensor, perm: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[:, j] = x[:, perm[j]]`` for a 16-bit matrix (``permute_cols`` of the reference)."""
    if out is None:
        out = torch.empty_like(x)
    if not x.is_cuda:
        out.copy_(x[:, perm.long()])
        return out
    assert x.element_size() == 2 and perm.dtype == torch.int32 and perm.numel() == x.shape[1]
    _native.call("tw_permute_cols", x.data_ptr(), out.data_ptr(), perm.data_ptr(), x.shape[0], x.shape[1],
                 _row_stride(x), _row_stride(out), _stream())
    return out


def copy_pages(cache: torch.Tensor, pairs: torch.Tensor) -> None:
    """Copies page ``pairs[i, 0]`` onto page ``pairs[i, 1]`` of one paged cache tensor ``[pages, ...]``
    (the copy-on-write step of csrc/cache_kernels.cu:69-130). ``pairs``: int64 ``[n, 2]``."""
    if pairs.numel() == 0:
        return
    if not cache.is_cuda:
        cache[pairs[:, 1].long()] = cache[pairs[:, 0].long()]
        return
    assert cache.is_contiguous() and pairs.dtype == torch.int64 and pairs.is_contiguous()
    pairs = pairs.to(cache.device)
    page_bytes = cache.stride(0) * cache.element_size()
    _native.call("tw_copy_pages", cache.data_ptr(), page_bytes, pairs.data_ptr(), pairs.shape[0], _stream())


def swap_pages(src: torch.Tensor, dst: torch.Tensor, pairs) -> None:
    """Copies page ``s`` of ``src`` to page ``d`` of ``dst`` for every ``(s, d)`` in ``pairs`` (host list);
    either tensor may live in pinned host memory (csrc/cache_kernels.cu:24-66). Consecutive pages
    travel as one asynchronous copy on the current stream."""
    pairs = [(int(s), int(d)) for s, d in pairs]
    if not pairs:
        return
    if not (src.is_cuda or dst.is_cuda):
        for s, d in pairs:
            dst[d].copy_(src[s])
        return
    assert src.is_contiguous() and dst.is_contiguous() and src.shape[1:] == dst.shape[1:] and src.dtype == dst.dtype
    import ctypes
    flat = (ctypes.c_longlong * (2 * len(pairs)))(*[v for p in pairs for v in p])
    page_bytes = src.stride(0) * src.element_size()
    _native.call("tw_swap_pages", src.data_ptr(), dst.data_ptr(), page_bytes, ctypes.addressof(flat), len(pairs),
                 _stream())


def merge_attn_states(a_out: torch.Tensor, a_lse: torch.Tensor, b_out: torch.Tensor, b_lse: torch.Tensor,
                      out: Optional[torch.Tensor] = None, want_lse: bool = False):
    """Merges two partial attention results over disjoint key sets (csrc/attention/merge_attn_states.cu).
    Outputs ``[T, H, D]`` bf16, log-sum-exps ``[H, T]`` fp32. Returns ``out`` or ``(out, lse)``."""
    T, H, D = a_out.shape
    if out is None:
        out = torch.empty_like(a_out)
    if not a_out.is_cuda:
        o, lse = reference.merge_attn_states(a_out, a_lse, b_out, b_lse)
        out.copy_(o)
        return (out, lse) if want_lse else out
    _check_bf16(a_out, b_out, out)
    assert a_out.is_contiguous() and b_out.is_contiguous() and out.is_contiguous()
    assert a_lse.dtype == torch.float32 and b_lse.dtype == torch.float32 and a_lse.is_contiguous() and b_lse.is_contiguous()
    lse = torch.empty(H, T, dtype=torch.float32, device=a_out.device) if want_lse else None
    _native.call("tw_merge_attn_states", out.data_ptr(), _p(lse), a_out.data_ptr(), a_lse.data_ptr(),
                 b_out.data_ptr(), b_lse.data_ptr(), T, H, D, _stream())
    return (out, lse) if want_lse else out


def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, vocab_start: int = 0,
              vocab_end: Optional[int] = None) -> torch.Tensor:
    T = ids.shape[0]
    H = table.shape[1]
    vocab_end = vocab_start + table.shape[0] if vocab_end is None else vocab_end
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    if not table.is_cuda:
        out.copy_(reference.embedding(ids, table, vocab_start, vocab_end))
        return out
    _check_bf16(table, out)
    assert ids.dtype == torch.int32
    _native.call("tw_embedding", ids.data_ptr(), table.data_ptr(), out.data_ptr(), _row_stride(out), T, H,
                 vocab_start, vocab_end, _stream())
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Row-wise argmax of fp32 logits -> int32 ids."""
    if not logits.is_cuda:
        return torch.argmax(logits, dim=-1).to(torch.int32)
    assert logits.dtype == torch.float32
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _native.call("tw_argmax", logits.data_ptr(), _row_stride(logits), out.data_ptr(), rows, V, _stream())
    return out


def pack_sample_params(temperature, top_k, top_p, min_p, seeds) -> torch.Tensor:
    """Host-side record array for :func:`sample`: one 32-byte record per row
    ``{f32 temperature, i32 top_k, f32 top_p, f32 min_p, u64 seed, u64 pad}`` as an int32 ``[B, 8]`` tensor."""
    import numpy as np
    B = len(temperature)
    rec = np.zeros(B, dtype=np.dtype([("t", "<f4"), ("k", "<i4"), ("p", "<f4"), ("m", "<f4"), ("s", "<u8"), ("z", "<u8")]))
    rec["t"], rec["k"], rec["p"], rec["m"] = temperature, top_k, top_p, min_p
    rec["s"] = np.asarray([int(s) & 0xFFFFFFFFFFFFFFFF for s in seeds], dtype=np.uint64)
    return torch.from_numpy(rec.view(np.int32).reshape(B, 8))


def sample(logits: torch.Tensor, packed_params: torch.Tensor) -> torch.Tensor:
    """One token per row of fp32 ``logits`` under per-row temperature / top-k / top-p / min-p and seed
    (``packed_params`` from :func:`pack_sample_params`, on the logits' device). CUDA only."""
    assert logits.is_cuda and logits.dtype == torch.float32 and packed_params.is_cuda
    rows, V = logits.shape
    assert packed_params.shape == (rows, 8) and packed_params.dtype == torch.int32 and packed_params.is_contiguous()
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _native.call("tw_sample", logits.data_ptr(), _row_stride(logits), rows, V, packed_params.data_ptr(), out.data_ptr(),
                 _stream())
    return out


# ---------------------------------------------------------------------------------------------
def attn_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                 cu_q: torch.Tensor, kv_lens: torch.Tensor, block_table: torch.Tensor, tile_seq: torch.Tensor,
                 tile_q0: torch.Tensor, num_tiles: int, hq: int, hkv: int, head_dim: int, scale: float,
                 max_ctas: int = 0, window: int = 0, softcap: float = 0.0) -> None:
    """Tensor-core causal attention for the 128-query tiles listed in (tile_seq, tile_q0), heaviest tile first.
    ``max_ctas`` bounds the SMs the persistent kernel occupies (0: all). ``window`` > 0: sliding-window
    attention, a query at position p sees keys (p - window, p]; ``softcap`` > 0: scores pass through
    ``cap * tanh(s / cap)`` (the options of vllm/v1/attention/backends/flash_attn.py:517-538)."""
    if num_tiles == 0:
        return
    _check_bf16(q, k_cache, v_cache, out)
    num_blocks, page = k_cache.shape[0], k_cache.shape[1]
    _native.call("tw_attn_prefill", q.data_ptr(), _row_stride(q), q.shape[0], k_cache.data_ptr(),
                 v_cache.data_ptr(), num_blocks, page, out.data_ptr(), _row_stride(out), cu_q.data_ptr(),
                 kv_lens.data_ptr(), block_table.data_ptr(), block_table.shape[1], tile_seq.data_ptr(),
                 tile_q0.data_ptr(), num_tiles, hq, hkv, head_dim, scale, max_ctas, int(window), float(softcap),
                 status_word(q.device).data_ptr(), _stream())


_decode_ws: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


# Decode attention kernel: "tc" (attn_decode_tc.cu: tcgen05; used for grouped-query models with head size 128
# once a sequence of the step has 256 keys, 1.4 to 1.8 times faster than the SIMT kernel on B200) or "simt"
# (attn_decode.cu, every other case). TW_DECODE_TC=0 forces "simt". "tcp" is the persistent form of "tc"
# (one CTA per SM walks the work items; TW_DECODE_TC=persistent): as fast or faster only for short contexts and
# models with 8 KV heads per GPU, so nothing selects it by default.
def _env_decode_variant() -> str:
    v = os.environ.get("TW_DECODE_TC", "1")
    return "tcp" if v == "persistent" else "tc" if v == "1" else "simt"


_decode_variant = _env_decode_variant()


def set_decode_variant(name: Optional[str]) -> None:
    """``"tc"`` / ``"tcp"`` / ``"simt"``; None restores the environment's choice."""
    global _decode_variant
    if name not in (None, "tc", "tcp", "simt"):
        raise ValueError(name)
    _decode_variant = name or _env_decode_variant()


def decode_splits(n_tok: int, hkv: int, max_kv_len: int, sm_count: int = 148) -> int:
    """How many ways the keys are split so that a small decode batch still fills the machine."""
    ctas = n_tok * hkv
    want = 8 * sm_count          # 4-warp CTAs: eight per SM hide the cache-line latency of the key walk
    if ctas == 0 or ctas >= want or max_kv_len <= 512:
        return 1
    return max(1, min(32, (want + ctas - 1) // ctas, (max_kv_len + 255) // 256))


def decode_splits_tc(ctas: int, tiles: int, sm_count: int = 148) -> int:
    """Split count for the tensor-core decode kernel (one CTA per SM at a time). Cost of a choice in units of
    one 128-key tile: waves x (fixed CTA cost of about three tiles + tiles per CTA), plus the merge pass when the
    keys are split; the cheapest wins. Whole waves matter: 64 CTAs of 64 tiles are best cut in two (one wave
    of 128 CTAs, measured 83 us) and not in three (two waves, 105 us)."""
    best, best_cost = 1, None
    for s in range(1, max(1, min(32, tiles)) + 1):
        waves = (ctas * s + sm_count - 1) // sm_count
        cost = waves * (3.0 + (tiles + s - 1) // s) + (2.0 if s > 1 else 0.0)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def decode_plan(n_tok: int, hq: int, hkv: int, head_dim: int, page: int, max_kv_len: int,
                sm_count: int = 148, plain: bool = True) -> tuple[str, int]:
    """(kernel, key splits) for a decode launch: everything that shapes the launch besides the tensor sizes,
    so a CUDA-graph signature that includes it replays the launch it captured. ``plain`` is False under a
    sliding window or a soft cap, which only the SIMT kernel implements."""
    use_tc = (plain and _decode_variant in ("tc", "tcp") and head_dim == 128 and hq // hkv <= 16 and max_kv_len >= 256
              and 8 <= page <= 128 and 128 % page == 0)
    tiles = (max_kv_len + 127) // 128
    if use_tc and _decode_variant == "tcp":
        # persistent CTAs: items of about four key tiles balance the SMs without whole-wave effects
        ctas = n_tok * hkv
        return "tcp", 1 if ctas >= 6 * sm_count else max(1, min(tiles // 4, 32))
    if use_tc:
        return "tc", decode_splits_tc(n_tok * hkv, tiles, sm_count)
    return "simt", decode_splits(n_tok, hkv, max_kv_len, sm_count)


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                tok_row: torch.Tensor, tok_seq: torch.Tensor, tok_kvlen: torch.Tensor, n_tok: int,
                block_table: torch.Tensor, hq: int, hkv: int, head_dim: int, scale: float, max_kv_len: int,
                sm_count: int = 148, window: int = 0, softcap: float = 0.0) -> None:
    """Single-query attention for the listed tokens; splits the keys when the grid would be small.
    ``window`` / ``softcap`` as in :func:`attn_prefill`."""
    if n_tok == 0:
        return
    _check_bf16(q, k_cache, v_cache, out)
    page = k_cache.shape[1]
    plain = window <= 0 and softcap <= 0
    kernel, splits = decode_plan(n_tok, hq, hkv, head_dim, page, min(max_kv_len, window) if window > 0 else max_kv_len,
                                 sm_count, plain)
    part_o = part_ml = None
    if splits > 1:
        # Partial results live in buffers whose sizes are powers of two and which are never freed: a captured
        # CUDA graph keeps the raw addresses, so a buffer may not go away while any graph could replay, and
        # rounding keeps the number of buffers small (launches of one stream use them one after the other).
        partials = 1 << max(0, (n_tok * hq * splits - 1).bit_length())
        key = (q.device.index, partials, head_dim)
        ws = _decode_ws.get(key)
        if ws is None:
            ws = (torch.empty(partials * head_dim, dtype=torch.float32, device=q.device),
                  torch.empty(partials * 2, dtype=torch.float32, device=q.device))
            _decode_ws[key] = ws
        part_o, part_ml = ws
    if kernel == "tc":
        _native.call("tw_attn_decode_tc", q.data_ptr(), _row_stride(q), k_cache.data_ptr(), v_cache.data_ptr(),
                     k_cache.shape[0], page, out.data_ptr(), _row_stride(out), tok_row.data_ptr(), tok_seq.data_ptr(),
                     tok_kvlen.data_ptr(), n_tok, block_table.data_ptr(), block_table.shape[1], hq, hkv, head_dim,
                     scale, splits, _p(part_o), _p(part_ml), status_word(q.device).data_ptr(), _stream())
        return
    if kernel == "tcp":
        _native.call("tw_attn_decode_tc_persistent", q.data_ptr(), _row_stride(q), k_cache.data_ptr(),
                     v_cache.data_ptr(), k_cache.shape[0], page, out.data_ptr(), _row_stride(out), tok_row.data_ptr(),
                     tok_seq.data_ptr(), tok_kvlen.data_ptr(), n_tok, block_table.data_ptr(), block_table.shape[1], hq,
                     hkv, head_dim, scale, splits, _p(part_o), _p(part_ml), sm_count if sm_count != 148 else 0,
                     status_word(q.device).data_ptr(), _stream())
        return
    _native.call("tw_attn_decode", q.data_ptr(), _row_stride(q), k_cache.data_ptr(), v_cache.data_ptr(), page,
                 out.data_ptr(), _row_stride(out), tok_row.data_ptr(), tok_seq.data_ptr(), tok_kvlen.data_ptr(),
                 n_tok, block_table.data_ptr(), block_table.shape[1], hq, hkv, head_dim, scale, splits,
                 _p(part_o), _p(part_ml), int(window), float(softcap), _stream())


# ---------------------------------------------------------------------------------------------
def moe_router(x: torch.Tensor, gate_w: torch.Tensor, topk: int, renormalize: bool = True,
               want_logits: bool = False):
    """Gate GEMV + softmax + top-k (+ renormalise). Returns (weights fp32 [T,k], ids int32 [T,k], logits|None)."""
    if not x.is_cuda:
        w, ids, logits = reference.moe_router(x, gate_w, topk, renormalize)
        return w, ids, (logits if want_logits else None)
    _check_bf16(x, gate_w)
    T, H = x.shape
    E = gate_w.shape[0]
    w = torch.empty(T, topk, dtype=torch.float32, device=x.device)
    ids = torch.empty(T, topk, dtype=torch.int32, device=x.device)
    logits = torch.empty(T, E, dtype=torch.float32, device=x.device) if want_logits else None
    _native.call("tw_moe_router", x.data_ptr(), _row_stride(x), gate_w.data_ptr(), w.data_ptr(), ids.data_ptr(),
                 _p(logits), T, H, E, topk, int(renormalize), _stream())
    return w, ids, logits


def moe_align(topk_ids: torch.Tensor, num_experts: int, tile_rows: int, expert_offsets: torch.Tensor,
              expert_cursor: torch.Tensor, tile_expert: torch.Tensor, meta: torch.Tensor) -> None:
    """Counting sort bookkeeping: padded expert offsets, expert per row tile, meta = [tiles, padded rows]."""
    _native.call("tw_moe_align", topk_ids.data_ptr(), topk_ids.numel(), num_experts, tile_rows,
                 expert_offsets.data_ptr(), expert_cursor.data_ptr(), tile_expert.data_ptr(),
                 tile_expert.numel(), meta.data_ptr(), _stream())


def moe_scatter(x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, expert_offsets: torch.Tensor,
                expert_cursor: torch.Tensor, a_sorted: torch.Tensor, row_scale: torch.Tensor,
                sorted_pos: torch.Tensor, num_experts: int) -> None:
    T, H = x.shape
    topk = topk_ids.shape[1]
    _native.call("tw_moe_scatter", x.data_ptr(), _row_stride(x), topk_ids.data_ptr(), topk_w.data_ptr(),
                 expert_offsets.data_ptr(), expert_cursor.data_ptr(), a_sorted.data_ptr(), row_scale.data_ptr(),
                 sorted_pos.data_ptr(), T * topk, topk, H, num_experts, _stream())


def moe_combine(y_sorted: torch.Tensor, sorted_pos: torch.Tensor, out: torch.Tensor, topk: int) -> None:
    T, H = out.shape
    _native.call("tw_moe_combine", y_sorted.data_ptr(), sorted_pos.data_ptr(), out.data_ptr(), _row_stride(out),
                 T, topk, H, _stream())
