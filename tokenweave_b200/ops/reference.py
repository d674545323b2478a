"""Plain PyTorch reference implementations of every op in :mod:`tokenweave_b200.ops`.

These are the oracle for the CUDA kernels (computed in fp32, rounded where the kernels round) and
the execution path on CPU, where the engine runs for tests and for the fp32 correctness
configuration. They follow the numerics order of the reference kernels
(csrc/layernorm_kernels.cu:87-113, csrc/tokenweave_fused_kernels.cu:127-151): the residual add is
done in the storage dtype, the sum of squares in fp32 over the rounded sums, the normalised value
is rounded to the storage dtype before the weight multiply.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------------
# norms
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * inv).to(x.dtype) * weight.to(x.dtype)


def add_rmsnorm_(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """In place: ``x += residual; residual = x; x = rmsnorm(x) * w``."""
    s = x + residual
    residual.copy_(s)
    x.copy_(rmsnorm(s, weight, eps))


def rmsnorm_copy_(x: torch.Tensor, residual_out: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """In place: ``residual_out = x; x = rmsnorm(x) * w``."""
    residual_out.copy_(x)
    x.copy_(rmsnorm(x, weight, eps))


# ---------------------------------------------------------------------------------------------
# linear algebra
def gemm(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
         row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a @ w.T`` with fp32 accumulation, optional bias (per column) and row scale."""
    out = a.float() @ w.float().t()
    if bias is not None:
        out = out + bias.float()
    if row_scale is not None:
        out = out * row_scale.float().unsqueeze(-1)
    return out.to(a.dtype)


def swiglu(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    xf = x.float()
    return (F.silu(xf[..., :d]) * xf[..., d:]).to(x.dtype)


FP8_MAX = 448.0


def quant_int8(x: torch.Tensor, scale: Optional[torch.Tensor] = None):
    """(int8 tensor, scales): symmetric, per-token ``max|row| / 127`` when ``scale`` is None, else the given scalar;
    round to nearest even and saturate."""
    xf = x.float()
    if scale is None:
        s = (xf.abs().amax(dim=-1) / 127.0).clamp_min(1e-10)
        q = torch.round(xf * s.reciprocal().unsqueeze(-1)).clamp(-128, 127).to(torch.int8)
        return q, s
    q = torch.round(xf * scale.float().reshape(()).reciprocal()).clamp(-128, 127).to(torch.int8)
    return q, scale


def gather_cache(cache: torch.Tensor, block_table: torch.Tensor, seq_lens: Sequence[int]) -> torch.Tensor:
    """Rows of every sequence, in block-table order, concatenated: ``[sum(seq_lens), kv_heads, D]``."""
    page = cache.shape[1]
    parts = []
    for b, n in enumerate(seq_lens):
        blocks = block_table[b, : (n + page - 1) // page].long()
        parts.append(cache.index_select(0, blocks).reshape(-1, *cache.shape[2:])[:n])
    return torch.cat(parts, 0) if parts else cache.new_zeros((0, *cache.shape[2:]))


def quant_fp8(x: torch.Tensor, scale: Optional[torch.Tensor] = None):
    """(e4m3 tensor, scales): per-token ``max|row| / 448`` when ``scale`` is None, else the given scalar."""
    xf = x.float()
    # x * (1 / scale): one reciprocal per row and a multiply per element, the arithmetic of the kernels
    # (bf16 inputs sit on e4m3 rounding ties often enough for the last ulp of the quotient to matter)
    if scale is None:
        s = (xf.abs().amax(dim=-1) / torch.tensor(FP8_MAX, dtype=torch.float32, device=x.device)).clamp_min(1e-10)
        q = (xf * s.reciprocal().unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
        return q, s
    q = (xf * scale.float().reshape(()).reciprocal()).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def gemm_fp8(a: torch.Tensor, w: torch.Tensor, a_scale: Optional[torch.Tensor], w_scale: Optional[torch.Tensor],
             bias: Optional[torch.Tensor] = None, swiglu: bool = False) -> torch.Tensor:
    """fp32 product of the dequantised operands, scaled per row and per output channel, rounded once."""
    acc = a.float() @ w.float().t()
    if a_scale is not None:
        acc = acc * a_scale.float().unsqueeze(-1)
    if w_scale is not None:
        acc = acc * w_scale.float().unsqueeze(0)
    if swiglu:
        n = acc.shape[1] // 2
        return (F.silu(acc[:, :n]) * acc[:, n:]).to(torch.bfloat16)
    if bias is not None:
        acc = acc + bias.float()
    return acc.to(torch.bfloat16)


def gemm_int8(a: torch.Tensor, w: torch.Tensor, a_scale: Optional[torch.Tensor], w_scale: Optional[torch.Tensor],
              bias: Optional[torch.Tensor] = None, swiglu: bool = False) -> torch.Tensor:
    """Exact integer product of int8 operands (accumulated in float64, which holds every partial sum exactly),
    scaled per row and per output channel in fp32 like the kernel's epilogue, rounded once."""
    acc = (a.double() @ w.double().t()).float()
    if a_scale is not None:
        acc = acc * a_scale.float().unsqueeze(-1)
    if w_scale is not None:
        acc = acc * w_scale.float().unsqueeze(0)
    if swiglu:
        n = acc.shape[1] // 2
        return (F.silu(acc[:, :n]) * acc[:, n:]).to(torch.bfloat16)
    if bias is not None:
        acc = acc + bias.float()
    return acc.to(torch.bfloat16)


ACTIVATION_KINDS = {"silu_and_mul": 0, "gelu_and_mul": 1, "gelu_tanh_and_mul": 2, "mul_and_silu": 3,
                    "fatrelu_and_mul": 4, "gelu_new": 5, "gelu_fast": 6, "quick_gelu": 7, "gelu": 8, "silu": 9}


def activation(x: torch.Tensor, kind: str, param: float = 0.0) -> torch.Tensor:
    """The activation functions of vllm/model_executor/layers/activation.py in fp32, rounded once."""
    xf = x.float()
    if ACTIVATION_KINDS[kind] <= 4:
        d = x.shape[-1] // 2
        a, b = xf[..., :d], xf[..., d:]
        if kind == "silu_and_mul":
            y = F.silu(a) * b
        elif kind == "gelu_and_mul":
            y = F.gelu(a) * b
        elif kind == "gelu_tanh_and_mul":
            y = F.gelu(a, approximate="tanh") * b
        elif kind == "mul_and_silu":
            y = a * F.silu(b)
        else:
            y = torch.where(a > param, a, torch.zeros_like(a)) * b
    elif kind == "gelu_new":
        y = F.gelu(xf, approximate="tanh")
    elif kind == "gelu_fast":
        y = 0.5 * xf * (1.0 + torch.tanh(xf * 0.7978845608 * (1.0 + 0.044715 * xf * xf)))
    elif kind == "quick_gelu":
        y = xf * torch.sigmoid(1.702 * xf)
    elif kind == "gelu":
        y = F.gelu(xf)
    else:
        y = F.silu(xf)
    return y.to(x.dtype)


def merge_attn_states(a_out: torch.Tensor, a_lse: torch.Tensor, b_out: torch.Tensor, b_lse: torch.Tensor):
    """Merge two partial attention results over disjoint key sets. Outputs ``[T, H, D]``, log-sum-exps
    ``[H, T]`` (natural log). Returns (merged output, merged lse)."""
    la = torch.where(torch.isinf(a_lse), torch.full_like(a_lse, -math.inf), a_lse).float()
    lb = torch.where(torch.isinf(b_lse), torch.full_like(b_lse, -math.inf), b_lse).float()
    m = torch.maximum(la, lb)
    safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    ea, eb = torch.exp(la - safe), torch.exp(lb - safe)
    tot = ea + eb
    wa = torch.where(tot > 0, ea / tot, torch.zeros_like(tot)).t().unsqueeze(-1)
    wb = torch.where(tot > 0, eb / tot, torch.zeros_like(tot)).t().unsqueeze(-1)
    out = (a_out.float() * wa + b_out.float() * wb).to(a_out.dtype)
    lse = torch.where(tot > 0, safe + torch.log(tot), torch.full_like(tot, -math.inf))
    return out, lse


def gemm_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(a @ Wg.T) * (a @ Wu.T)`` where ``w_gate_up = [Wg; Wu]``, rounded once at the end."""
    inter = w_gate_up.shape[0] // 2
    y = a.float() @ w_gate_up.float().t()
    out = F.silu(y[:, :inter]) * y[:, inter:]
    if row_scale is not None:
        out = out * row_scale.float().unsqueeze(-1)
    return out.to(a.dtype)


# ---------------------------------------------------------------------------------------------
# rotary embedding and KV cache
def build_cos_sin_cache(head_dim: int, max_pos: int, theta: float,
                        rope_scaling: Optional[dict] = None, device="cpu") -> torch.Tensor:
    """fp32 table ``[max_pos, head_dim]``: cos in the first half of each row, sin in the second.

    ``rope_scaling`` supports the Llama-3 frequency rescaling
    (vllm/model_executor/layers/rotary_embedding.py:808-851), linear position scaling (:184-260),
    dynamic NTK scaling evaluated at the extended length (:263-343) and YaRN (:346-440: per-frequency
    blend of interpolated and extrapolated frequencies plus the attention-temperature factor that
    multiplies cos and sin). All variants only change this table; the rotary kernel is the same.
    """
    half = head_dim // 2
    exponents = torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim
    inv_freq = 1.0 / (theta ** exponents)
    mscale = 1.0
    if rope_scaling:
        kind = rope_scaling.get("rope_type", rope_scaling.get("type", "default"))
        if kind in ("default", "", None):
            pass
        elif kind == "dynamic":
            factor = float(rope_scaling["factor"])
            orig = float(rope_scaling.get("original_max_position_embeddings", max_pos / factor))
            base = theta * ((factor * (orig * factor) / orig) - (factor - 1)) ** (head_dim / (head_dim - 2))
            inv_freq = 1.0 / (base ** exponents)
        elif kind == "yarn":
            factor = float(rope_scaling["factor"])
            orig = float(rope_scaling.get("original_max_position_embeddings", max_pos / factor))
            beta_fast = float(rope_scaling.get("beta_fast", 32))
            beta_slow = float(rope_scaling.get("beta_slow", 1))

            def corr_dim(rot):      # the dimension whose wavelength makes `rot` turns over the original length
                return head_dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(theta))
            lo = max(math.floor(corr_dim(beta_fast)), 0)
            hi = min(math.ceil(corr_dim(beta_slow)), head_dim - 1)
            if rope_scaling.get("truncate", True) is False:
                lo, hi = max(corr_dim(beta_fast), 0), min(corr_dim(beta_slow), head_dim - 1)
            if lo == hi:
                hi += 0.001
            ramp = ((torch.arange(half, dtype=torch.float64) - lo) / (hi - lo)).clamp(0, 1)
            extrap = 1.0 - ramp                                   # 1 where the frequency is kept as is
            inv_freq = inv_freq / factor * (1 - extrap) + inv_freq * extrap
            att = rope_scaling.get("attention_factor")
            mscale = float(att) if att is not None else (0.1 * math.log(factor) + 1.0 if factor > 1 else 1.0)
        elif kind == "llama3":
            factor = float(rope_scaling["factor"])
            low = float(rope_scaling.get("low_freq_factor", 1.0))
            high = float(rope_scaling.get("high_freq_factor", 4.0))
            orig = float(rope_scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = (orig / wavelen - low) / (high - low)
            scaled = torch.where(
                wavelen < orig / high, inv_freq,
                torch.where(wavelen > orig / low, inv_freq / factor,
                            (1 - smooth) * inv_freq / factor + smooth * inv_freq))
            inv_freq = scaled
        elif kind == "linear":
            inv_freq = inv_freq / float(rope_scaling["factor"])
        elif kind in ("longrope", "su"):
            # Phi-3 LongRoPE (vllm/model_executor/layers/rotary_embedding.py ``Phi3LongRoPEScaledRotaryEmbedding``):
            # per-frequency rescale factors, one list for contexts inside the original window and one beyond it.
            # Both tables are stored back to back - rows [0, original) "short", rows [original, original + max_pos)
            # "long" - and ``longrope_offset`` tells the runner by how much to shift the positions of a step that
            # reaches beyond the original window.
            orig = int(rope_scaling.get("original_max_position_embeddings", max_pos))
            scale = max_pos / orig
            mscale = 1.0 if scale <= 1.0 else math.sqrt(1.0 + math.log(scale) / math.log(orig))
            att = rope_scaling.get("attention_factor")
            if att is not None:
                mscale = float(att)
            if "short_factor" not in rope_scaling or "long_factor" not in rope_scaling:
                raise ValueError("longrope needs the short_factor and long_factor lists")
            tables = []
            for factors, rows in ((rope_scaling["short_factor"], orig), (rope_scaling["long_factor"], max_pos)):
                f = torch.tensor(factors, dtype=torch.float64)
                if f.numel() != half:
                    raise ValueError(f"longrope factor lists need {half} entries, got {f.numel()}")
                fr = torch.outer(torch.arange(rows, dtype=torch.float64), inv_freq / f)
                tables.append(torch.cat([fr.cos(), fr.sin()], dim=-1) * mscale)
            return torch.cat(tables, 0).float().to(device)
        else:
            raise ValueError(f"unsupported rope_scaling type {kind!r} (default, linear, dynamic, yarn, llama3, longrope)")
    t = torch.arange(max_pos, dtype=torch.float64)
    freqs = torch.outer(t, inv_freq)
    return (torch.cat([freqs.cos(), freqs.sin()], dim=-1) * mscale).float().to(device)


def longrope_offset(rope_scaling: Optional[dict], max_pos: int) -> int:
    """Rows to add to the positions of a step that reaches beyond the original context window (0 for every
    other rope variant): the "long" table starts there."""
    if not rope_scaling or rope_scaling.get("rope_type", rope_scaling.get("type")) not in ("longrope", "su"):
        return 0
    return int(rope_scaling.get("original_max_position_embeddings", max_pos))


def rope_kv_write_(qkv: torch.Tensor, positions: torch.Tensor, slots: Optional[torch.Tensor],
                   cos_sin: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                   hq: int, hkv: int, head_dim: int, write_k_back: bool = True,
                   qk_norm: Optional[tuple] = None) -> None:
    """NeoX rotary on the q and k heads of ``qkv`` ([T, (hq+2*hkv)*D]) in place, then scatter the
    rotated k and the v rows into the paged caches ([blocks, page, hkv, D]) at ``slots``
    (negative slots are skipped). ``qk_norm = (q_weight, k_weight, eps)``: RMSNorm over ``head_dim`` of
    every q and k head before the rotation (vllm/model_executor/models/qwen3.py ``q_norm`` / ``k_norm``)."""
    T = qkv.shape[0]
    if T == 0:
        return
    D = head_dim
    half = D // 2
    cs = cos_sin.index_select(0, positions.long())
    cos = cs[:, :half].unsqueeze(1)
    sin = cs[:, half:].unsqueeze(1)
    qk = qkv[:, : (hq + hkv) * D].reshape(T, hq + hkv, D).float()
    if qk_norm is not None:
        qw, kw, eps = qk_norm
        w = torch.cat([qw.float().expand(hq, D), kw.float().expand(hkv, D)], 0)
        qk = qk * torch.rsqrt(qk.pow(2).mean(-1, keepdim=True) + eps) * w
        if qkv.dtype != torch.float32:      # the kernel rounds the normalised head to the storage type once
            qk = qk.to(qkv.dtype).float()
    x, y = qk[..., :half], qk[..., half:]
    rot = torch.cat([x * cos - y * sin, y * cos + x * sin], dim=-1).to(qkv.dtype)
    k_rot = rot[:, hq:]
    qkv[:, : hq * D] = rot[:, :hq].reshape(T, hq * D)
    if write_k_back:
        qkv[:, hq * D: (hq + hkv) * D] = k_rot.reshape(T, hkv * D)
    if slots is not None and k_cache is not None:
        valid = slots >= 0
        idx = slots[valid].long()
        kc = k_cache.view(-1, hkv, D)
        vc = v_cache.view(-1, hkv, D)
        kc[idx] = k_rot[valid]
        vc[idx] = qkv[:, (hq + hkv) * D:].reshape(T, hkv, D)[valid]


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0,
              vocab_end: Optional[int] = None) -> torch.Tensor:
    vocab_end = vocab_start + table.shape[0] if vocab_end is None else vocab_end
    ok = (ids >= vocab_start) & (ids < vocab_end)
    local = torch.where(ok, ids - vocab_start, torch.zeros_like(ids)).long()
    out = table.index_select(0, local)
    return out * ok.unsqueeze(-1).to(out.dtype)


# ---------------------------------------------------------------------------------------------
# attention
def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: Sequence[int],
                    kv_lens: Sequence[int], block_table: torch.Tensor, hq: int, hkv: int, head_dim: int,
                    scale: float, window: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """Causal varlen attention over a paged cache. ``q``: [T, hq*D]; caches [blocks, page, hkv, D];
    sequence b owns query rows ``cu_q[b]:cu_q[b+1]`` whose last row sees ``kv_lens[b]`` keys. ``window`` > 0:
    a query at position p sees keys (p - window, p] only; ``softcap`` > 0: scores become
    ``softcap * tanh(score / softcap)`` before the softmax."""
    T = q.shape[0]
    D = head_dim
    page = k_cache.shape[1]
    out = torch.zeros(T, hq * D, dtype=q.dtype, device=q.device)
    group = hq // hkv
    for b in range(len(kv_lens)):
        qs, qe = int(cu_q[b]), int(cu_q[b + 1])
        q_len = qe - qs
        if q_len <= 0:
            continue
        kv_len = int(kv_lens[b])
        n_pages = (kv_len + page - 1) // page
        blocks = block_table[b, :n_pages].long()
        k = k_cache.index_select(0, blocks).reshape(-1, hkv, D)[:kv_len].float()
        v = v_cache.index_select(0, blocks).reshape(-1, hkv, D)[:kv_len].float()
        qb = q[qs:qe].reshape(q_len, hq, D).float()
        k = k.repeat_interleave(group, dim=1)
        v = v.repeat_interleave(group, dim=1)
        s = torch.einsum("qhd,khd->hqk", qb, k) * scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        qpos = torch.arange(kv_len - q_len, kv_len, device=q.device).unsqueeze(-1)
        kpos = torch.arange(kv_len, device=q.device).unsqueeze(0)
        hidden_keys = kpos > qpos
        if window > 0:
            hidden_keys = hidden_keys | (kpos <= qpos - window)
        s = s.masked_fill(hidden_keys.unsqueeze(0), float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hqk,khd->qhd", p, v)
        out[qs:qe] = o.reshape(q_len, hq * D).to(q.dtype)
    return out


# ---------------------------------------------------------------------------------------------
# mixture of experts
def moe_router(x: torch.Tensor, gate_w: torch.Tensor, topk: int, renormalize: bool = True):
    """Returns (weights [T, k] fp32, ids [T, k] int32, logits [T, E] fp32)."""
    logits = x.float() @ gate_w.float().t()
    probs = torch.softmax(logits, dim=-1)
    w, ids = torch.topk(probs, topk, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32), logits


def moe_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor,
                topk_ids: torch.Tensor) -> torch.Tensor:
    """Loop-over-experts MoE MLP: ``sum_k w_k * W2[e_k] (silu(W1[e_k] x) * W3[e_k] x)``.
    ``w13``: [E, 2*I, H] (gate rows first), ``w2``: [E, H, I]. The activation and the weighted
    expert output are rounded to the storage dtype, the top-k sum runs in fp32."""
    T, H = x.shape
    E = w13.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(E):
        sel = (topk_ids == e)
        tok, slot = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x.index_select(0, tok)
        act = gemm_swiglu(xe, w13[e])
        ye = gemm(act, w2[e], row_scale=topk_w[tok, slot])
        out.index_add_(0, tok, ye.float())
    return out.to(x.dtype)


# ---------------------------------------------------------------------------------------------
# fused collective (single-process emulation over a list of per-rank tensors)
def fused_allreduce_add_rmsnorm(partials: Sequence[torch.Tensor], residual: torch.Tensor, weight: torch.Tensor,
                                eps: float):
    """Reference of the fused RS + add + RMSNorm + AG: returns (normed [T,H], new residual [T,H]).
    The cross-rank sum accumulates in fp32 and is rounded to the storage dtype before the add."""
    acc = torch.zeros_like(partials[0], dtype=torch.float32)
    for p in partials:
        acc += p.float()
    s = acc.to(partials[0].dtype) + residual
    return rmsnorm(s, weight, eps), s
