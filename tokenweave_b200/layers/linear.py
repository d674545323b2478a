"""Tensor-parallel linear layers and their checkpoint loaders.

Counterpart of vllm/model_executor/layers/linear.py:373-1342. Weights keep the ``[out, in]`` layout
of HuggingFace checkpoints, which is exactly the K-major B operand of the tcgen05 GEMM, so nothing is
transposed at load time. ``RowParallelLinear`` never all-reduces: it writes its partial sums into the
caller's buffer (a slice of the symmetric staging buffer) and the fused collective that follows
reduces them (reference: ``apply_inplace``, linear.py:203-230 and :1290-1334).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..parallel.state import get_tp


def _param(*shape, dtype, device) -> nn.Parameter:
    return nn.Parameter(torch.empty(*shape, dtype=dtype, device=device), requires_grad=False)


class _QuantizableLinear(nn.Module):
    """Shared GEMM dispatch of the linear layers. After :meth:`quantize_fp8_` the bf16 weight is replaced
    by an e4m3 weight with one fp32 scale per output channel and every call quantises its input per
    token on the fly (dynamic activation scales) before the fp8 tcgen05 GEMM — the scheme of the
    reference's ``Fp8LinearMethod`` with dynamic activation quantisation
    (vllm/model_executor/layers/quantization/fp8.py) on its sm100 scaled-mm. :meth:`quantize_int8_` is the same
    scheme with symmetric int8 weights and activations and exact integer accumulation (the reference's
    compressed-tensors W8A8 int8 path on its CUTLASS int8 scaled-mm)."""

    weight_scale: Optional[torch.Tensor] = None

    def quantize_int8_(self) -> None:
        if self.weight_scale is not None:
            return
        q, scale = ops.quant_int8(self.weight.data)
        self.weight = nn.Parameter(q, requires_grad=False)
        self.weight_scale = scale

    def quantize_fp8_(self) -> None:
        if self.weight_scale is not None:
            return
        q, scale = ops.quant_fp8(self.weight.data)
        self.weight = nn.Parameter(q, requires_grad=False)
        self.weight_scale = scale

    def _gemm(self, x: torch.Tensor, out: Optional[torch.Tensor], *, bias=None, row_scale=None, swiglu=False,
              max_ctas: int = 0) -> torch.Tensor:
        if self.weight_scale is None:
            return ops.gemm(x, self.weight, out=out, bias=bias, row_scale=row_scale, swiglu=swiglu, max_ctas=max_ctas)
        if out is None:
            n = self.weight.shape[0] // 2 if swiglu else self.weight.shape[0]
            out = torch.empty(x.shape[0], n, dtype=x.dtype, device=x.device)
        if self.weight.dtype == torch.int8:
            xq, x_scale = ops.quant_int8(x, max_ctas=max_ctas)
            if row_scale is not None:
                x_scale = x_scale * row_scale
            return ops.gemm_int8(xq, self.weight, x_scale, self.weight_scale, out=out, bias=bias, swiglu=swiglu,
                                 max_ctas=max_ctas)
        xq, x_scale = ops.quant_fp8(x, max_ctas=max_ctas)
        if row_scale is not None:
            x_scale = x_scale * row_scale
        return ops.gemm_fp8(xq, self.weight, x_scale, self.weight_scale, out=out, bias=bias, swiglu=swiglu,
                            max_ctas=max_ctas)


class ReplicatedLinear(_QuantizableLinear):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, *, dtype, device):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = _param(out_features, in_features, dtype=dtype, device=device)
        self.bias = _param(out_features, dtype=dtype, device=device) if bias else None

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
        return self._gemm(x, out, bias=self.bias, max_ctas=max_ctas)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        param.data.copy_(loaded)


class ColumnParallelLinear(_QuantizableLinear):
    """Output features sharded over the TP ranks; the input is replicated."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, *, dtype, device):
        super().__init__()
        tp = get_tp()
        assert out_features % tp.world_size == 0
        self.in_features = in_features
        self.out_features = out_features
        self.out_per_rank = out_features // tp.world_size
        self.weight = _param(self.out_per_rank, in_features, dtype=dtype, device=device)
        self.bias = _param(self.out_per_rank, dtype=dtype, device=device) if bias else None

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
        return self._gemm(x, out, bias=self.bias, max_ctas=max_ctas)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        r = get_tp().rank
        param.data.copy_(loaded.narrow(0, r * self.out_per_rank, self.out_per_rank))


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several column-parallel projections packed along the output dim (gate_up_proj = [gate | up])."""

    def __init__(self, in_features: int, output_sizes: list[int], bias: bool = False, *, dtype, device):
        tp = get_tp()
        assert all(s % tp.world_size == 0 for s in output_sizes)
        super().__init__(in_features, sum(output_sizes), bias, dtype=dtype, device=device)
        self.output_sizes = output_sizes

    def forward_swiglu(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
        """silu(x @ gate.T) * (x @ up.T), fused into the GEMM epilogue."""
        return self._gemm(x, out, swiglu=True, max_ctas=max_ctas)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        tp = get_tp()
        if shard_id is None:   # already packed checkpoint
            off = 0
            for i, s in enumerate(self.output_sizes):
                self.weight_loader(param, loaded.narrow(0, off, s), i)
                off += s
            return
        size = self.output_sizes[shard_id] // tp.world_size
        dst_off = sum(self.output_sizes[:shard_id]) // tp.world_size
        param.data.narrow(0, dst_off, size).copy_(loaded.narrow(0, tp.rank * size, size))


class QKVParallelLinear(_QuantizableLinear):
    """Packed [q | k | v] projection; KV heads are replicated when tp > num_kv_heads
    (vllm/model_executor/layers/linear.py:856-897)."""

    def __init__(self, hidden: int, head_dim: int, num_q_heads: int, num_kv_heads: int, bias: bool = False, *,
                 dtype, device):
        super().__init__()
        tp = get_tp()
        assert num_q_heads % tp.world_size == 0
        self.head_dim = head_dim
        self.q_heads = num_q_heads // tp.world_size
        if tp.world_size >= num_kv_heads:
            assert tp.world_size % num_kv_heads == 0
            self.kv_heads, self.kv_replicas = 1, tp.world_size // num_kv_heads
        else:
            assert num_kv_heads % tp.world_size == 0
            self.kv_heads, self.kv_replicas = num_kv_heads // tp.world_size, 1
        self.out_per_rank = (self.q_heads + 2 * self.kv_heads) * head_dim
        self.weight = _param(self.out_per_rank, hidden, dtype=dtype, device=device)
        self.bias = _param(self.out_per_rank, dtype=dtype, device=device) if bias else None

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, max_ctas: int = 0) -> torch.Tensor:
        return self._gemm(x, out, bias=self.bias, max_ctas=max_ctas)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        tp = get_tp()
        D = self.head_dim
        if shard_id == "q":
            size, dst, src = self.q_heads * D, 0, tp.rank * self.q_heads * D
        else:
            size = self.kv_heads * D
            dst = self.q_heads * D + (0 if shard_id == "k" else size)
            src = (tp.rank // self.kv_replicas) * size
        param.data.narrow(0, dst, size).copy_(loaded.narrow(0, src, size))


class RowParallelLinear(_QuantizableLinear):
    """Input features sharded; the output holds this rank's partial sums (no all-reduce here)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, *, dtype, device):
        super().__init__()
        tp = get_tp()
        assert in_features % tp.world_size == 0
        self.in_features, self.out_features = in_features, out_features
        self.in_per_rank = in_features // tp.world_size
        self.weight = _param(out_features, self.in_per_rank, dtype=dtype, device=device)
        self.bias = _param(out_features, dtype=dtype, device=device) if bias else None

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, max_ctas: int = 0,
                row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        bias = self.bias if get_tp().rank == 0 else None   # added once across the reduction
        return self._gemm(x, out, bias=bias, row_scale=row_scale, max_ctas=max_ctas)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        r = get_tp().rank
        if param.dim() == 1:
            param.data.copy_(loaded)
        else:
            param.data.copy_(loaded.narrow(1, r * self.in_per_rank, self.in_per_rank))
