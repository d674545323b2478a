"""Tensor-parallel communicator: the fused reduce-scatter + residual-add + RMSNorm + all-gather and
the stand-alone collectives, over three transports.

* in-kernel NVLS multimem or peer loads/stores on a symmetric buffer (``csrc/comm_fused.cu``),
* NCCL through ``torch.distributed`` (the baseline the reference calls "ring"),
* gloo on CPU, where the fused op is emulated as all-reduce followed by add+RMSNorm (used by tests and
  by the fp32 correctness configuration).

Reference call sites: ``fused_allreduce_layernorm`` (vllm/model_executor/models/tokenweave_utils.py:24-92),
``multimem_all_reduce / reduce_scatter / all_gather`` (vllm/distributed/triton_comm/triton_comm.py:240-386),
``pytorch_all_reduce`` (vllm/distributed/communication_op.py:15-20).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _native
from .state import TPState, get_tp
from .symm_mem import SymmetricBuffer

# signal-pad slot ranges: independent call sites never share barrier slots
CHANNEL_FUSED = 0
CHANNEL_COLLECTIVE = 0
OP_ALL_REDUCE, OP_REDUCE_SCATTER, OP_ALL_GATHER = 0, 1, 2


class TPCommunicator:
    def __init__(self, buf: Optional[SymmetricBuffer], tp: Optional[TPState] = None, wait_budget_ms: int = 2000,
                 transport: str = "auto"):
        self.tp = tp or get_tp()
        self.buf = buf
        self.budget_ns = int(wait_budget_ms) * 1_000_000
        self.in_kernel = (buf is not None and buf.provider != "local" and self.tp.world_size > 1)
        self.use_mc = self.in_kernel and buf.has_multicast and transport in ("auto", "multimem")
        if transport == "multimem" and self.in_kernel and not buf.has_multicast:
            raise RuntimeError("multimem transport requested but the symmetric buffer has no multicast mapping")
        self.pynccl = None                      # NcclCommunicator of this group (enable_pynccl)
        self.custom_ar_enabled = False          # the "custom all-reduce" baseline may be used (enable_custom_all_reduce)
        self.custom_ar_max_bytes = 8 << 20
        self._car_out: Optional[torch.Tensor] = None

    # ---- library baselines --------------------------------------------------------------------
    def enable_pynccl(self) -> bool:
        """A private NCCL communicator (ctypes, ``parallel/pynccl.py``) for the library-only baseline and the
        logits gather: collectives go onto the current stream without the process-group layer, so they can
        be captured in CUDA graphs (vllm/distributed/device_communicators/pynccl.py:109-217). Collective:
        every rank of the group calls it. Returns False (and leaves ``torch.distributed`` in charge) on CPU,
        for one rank, or when the library cannot be loaded."""
        if self.pynccl is not None:
            return True
        if self.world == 1 or self.tp.device.type != "cuda":
            return False
        from .pynccl import NcclCommunicator
        from .state import broadcast_object
        try:
            self.pynccl = NcclCommunicator(self.tp.rank, self.world, self.tp.device, broadcast_object)
        except OSError:
            self.pynccl = None
        return self.pynccl is not None

    def enable_custom_all_reduce(self, max_bytes: int = 8 << 20) -> None:
        """Allows :meth:`custom_all_reduce_` to use peer loads / stores (the engine option
        ``disable_custom_all_reduce=False``)."""
        self.custom_ar_enabled = self.in_kernel
        self.custom_ar_max_bytes = max_bytes

    @property
    def world(self) -> int:
        return self.tp.world_size

    def _mc(self) -> Optional[int]:
        return self.buf.multicast_ptr if self.use_mc else None

    def reset_after_failure(self) -> None:
        """Collective recovery after a kernel reported a failed wait: every rank calls this together.

        A barrier that ran out leaves raised flags behind, a fused GEMM that gave up leaves tile counters and
        shard epochs half-way; the next kernel would read them as its own. All ranks drain their device, meet
        on the host, zero their signal pad, flag words, epochs and status word, and meet again before any
        kernel runs."""
        from .state import cpu_barrier
        if self.tp.device.type == "cuda":
            torch.cuda.synchronize(self.tp.device)
        cpu_barrier()
        if self.in_kernel:
            self.buf.reset_signal_pads()
            flags = getattr(self, "flags", None)
            if flags is not None:
                flags.tensor.zero_()
                flags.reset_signal_pads()
                self._epochs.zero_()
        if self.tp.device.type == "cuda":
            ops.reset_status(self.tp.device)
            torch.cuda.synchronize(self.tp.device)
        cpu_barrier()

    # ---- the product op -----------------------------------------------------------------
    def fused_allreduce_add_rmsnorm_(self, x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                                     eps: float, max_ctas: int = 16, mode: int = 0, rows_in_flight: int = 0) -> None:
        """``x`` ([T, H] rows of the symmetric buffer holding this rank's partial sums) becomes
        ``rmsnorm(sum_ranks(x) + residual) * weight`` on every rank; ``residual`` ([T, H], same row
        indexing as ``x``) is updated on this rank's shard of the rows only."""
        T, H = x.shape
        if self.world == 1:
            ops.add_rmsnorm_(x, residual, weight, eps, max_ctas=0)
            return
        if T % self.world != 0:
            raise ValueError(f"token count {T} must be a multiple of the TP size {self.world}")
        if not self.in_kernel:
            dist.all_reduce(x, group=self.tp.group)
            ops.add_rmsnorm_(x, residual, weight, eps)
            return
        rpr = T // self.world
        shard_res = residual[self.tp.rank * rpr:(self.tp.rank + 1) * rpr]
        _native.call("tw_fused_rs_norm_ag", self._mc(), self.buf.peer_ptrs_dev, self.buf.signal_pads_dev,
                     self.tp.rank, self.world, CHANNEL_FUSED, self.budget_ns,
                     ops.status_word(x.device).data_ptr(), self.buf.byte_offset(x), shard_res.data_ptr(),
                     shard_res.stride(0), weight.data_ptr(), T, H, eps, max_ctas, mode, rows_in_flight,
                     torch.cuda.current_stream().cuda_stream)

    # ---- stand-alone collectives on rows of the symmetric buffer ---------------------------
    def _collective(self, x: torch.Tensor, op: int, max_ctas: int, peer_only: bool = False) -> None:
        _native.call("tw_collective", None if peer_only else self._mc(), self.buf.peer_ptrs_dev, self.buf.signal_pads_dev, self.tp.rank,
                     self.world, CHANNEL_COLLECTIVE, self.budget_ns, ops.status_word(x.device).data_ptr(),
                     self.buf.byte_offset(x), x.numel() * x.element_size(), op, max_ctas,
                     torch.cuda.current_stream().cuda_stream)

    def all_reduce_(self, x: torch.Tensor, max_ctas: int = 16) -> None:
        if self.world == 1:
            return
        if self.in_kernel:
            self._collective(x, OP_ALL_REDUCE, max_ctas)
        else:
            dist.all_reduce(x, group=self.tp.group)

    def reduce_scatter_(self, x: torch.Tensor, max_ctas: int = 16) -> None:
        """In place: this rank's 1/world slice of ``x`` (by flat offset) becomes the reduced slice."""
        if self.world == 1:
            return
        if self.in_kernel:
            self._collective(x, OP_REDUCE_SCATTER, max_ctas)
        else:
            flat = x.view(-1)
            n = flat.numel() // self.world
            out = torch.empty(n, dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(out, flat, group=self.tp.group)
            flat[self.tp.rank * n:(self.tp.rank + 1) * n] = out

    def all_gather_(self, x: torch.Tensor, max_ctas: int = 16) -> None:
        """In place: every rank's slice of ``x`` is broadcast to all ranks."""
        if self.world == 1:
            return
        if self.in_kernel:
            self._collective(x, OP_ALL_GATHER, max_ctas)
        else:
            flat = x.view(-1)
            n = flat.numel() // self.world
            mine = flat[self.tp.rank * n:(self.tp.rank + 1) * n].clone()
            dist.all_gather_into_tensor(flat, mine, group=self.tp.group)

    def oneshot_all_reduce(self, x: torch.Tensor, out: torch.Tensor, max_ctas: int = 36) -> torch.Tensor:
        """Small-message peer all-reduce: every rank pulls the whole message from every peer."""
        if self.world == 1:
            out.copy_(x)
            return out
        if not self.in_kernel:
            out.copy_(x)
            dist.all_reduce(out, group=self.tp.group)
            return out
        _native.call("tw_oneshot_allreduce", self.buf.peer_ptrs_dev, self.buf.signal_pads_dev, self.tp.rank,
                     self.world, CHANNEL_COLLECTIVE, self.budget_ns, ops.status_word(x.device).data_ptr(),
                     self.buf.byte_offset(x), x.numel() * x.element_size(), out.data_ptr(), max_ctas,
                     torch.cuda.current_stream().cuda_stream)
        return out

    # ---- NCCL baseline ------------------------------------------------------------------
    def nccl_all_reduce_(self, x: torch.Tensor) -> None:
        if self.world == 1:
            return
        if self.pynccl is not None and x.is_contiguous():
            self.pynccl.all_reduce(x)
        else:
            dist.all_reduce(x, group=self.tp.group)

    def nccl_all_gather(self, out: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """``out`` ([world * n]) receives every rank's ``x`` ([n]) in rank order."""
        if self.pynccl is not None and x.is_contiguous() and out.is_contiguous():
            self.pynccl.all_gather(out, x)
        else:
            dist.all_gather_into_tensor(out, x, group=self.tp.group)
        return out

    # ---- custom all-reduce baseline ---------------------------------------------------------
    def custom_all_reduce_(self, x: torch.Tensor) -> None:
        """The reference's "custom all-reduce" (csrc/custom_all_reduce.cuh:296-364, size policy :558-589; Python
        side vllm/distributed/device_communicators/custom_all_reduce.py:48-301) for rows of the symmetric
        buffer, in place: peer loads and stores with a flag barrier, no NVLS. One-shot (every rank pulls the whole
        message from every peer) below 512 KiB for up to 4 ranks and below 256 KiB for up to 8, two-shot
        (reduce-scatter + all-gather over peer pointers) up to ``custom_ar_max_bytes``, NCCL beyond that or
        when the option is off. The reference registers the buffers of a captured graph with its peers
        (``register_graph_buffers``, custom_all_reduce.py:193); here the activations already live in symmetric
        memory every rank can address, so there is nothing to register and the calls replay from a graph as
        they are."""
        if self.world == 1:
            return
        nbytes = x.numel() * x.element_size()
        ok = (self.custom_ar_enabled and x.dtype == torch.bfloat16 and x.is_contiguous() and self.world in (2, 4, 6, 8)
              and nbytes <= self.custom_ar_max_bytes and nbytes % (16 * self.world) == 0)
        if not ok:
            self.nccl_all_reduce_(x)
            return
        one_shot = (self.world <= 4 and nbytes < 512 * 1024) or (self.world <= 8 and nbytes < 256 * 1024)
        if one_shot:
            if self._car_out is None:
                self._car_out = torch.empty(512 * 1024 // 2, dtype=torch.bfloat16, device=x.device)
            out = self._car_out[: x.numel()]
            self.oneshot_all_reduce(x, out)
            # every rank has read every peer's copy before any rank overwrites its own: the one-shot kernel
            # ends with a barrier
            x.view(-1).copy_(out)
        else:
            self._collective(x, OP_ALL_REDUCE, 36, peer_only=True)

    # ---- GEMM fused with its collective (one kernel each) ----------------------------------
    FLAG_WORDS_PER_REGION = 256      # 128 tile counters (+128 "done" counters share the range), then epochs

    def attach_flag_buffer(self, flags: "SymmetricBuffer") -> None:
        """A small zero-initialised symmetric buffer for the tile counters and shard epochs of the fused
        GEMM kernels (two regions: token subset 0 / unsplit, and subset 1)."""
        self.flags = flags
        self._flag_tables = {}
        self._epochs = torch.zeros(4, dtype=torch.int32, device=flags.tensor.device)

    def _flag_table(self, region: int, which: str) -> int:
        key = (region, which)
        t = self._flag_tables.get(key)
        if t is None:
            word = region * 512 + (0 if which == "tile" else 256)
            t = self.flags.pointer_table(word * 4)
            self._flag_tables[key] = t
        return t.data_ptr()

    def fused_gemm_available(self, rows_view: torch.Tensor) -> bool:
        T, H = rows_view.shape
        return (self.in_kernel and getattr(self, "flags", None) is not None and H <= 8192 and T % self.world == 0
                and T // self.world <= 128 * 128)

    def gemm_rs_norm_(self, a: torch.Tensor, w: torch.Tensor, out_rows: torch.Tensor, M: int, residual: torch.Tensor,
                      norm_w: torch.Tensor, eps: float, comm_ctas: int = 8, bias: Optional[torch.Tensor] = None,
                      region: int = 0, max_ctas: int = 0) -> None:
        """``out_rows`` ([T, H] rows of the symmetric buffer) receives this rank's partial sums
        ``a[:M] @ w.T``; when the kernel returns, this rank's shard of ``out_rows`` holds
        ``rmsnorm(sum over ranks + residual) * norm_w`` and its shard of ``residual`` is updated. Other rows
        of ``out_rows`` are stale until an all-gather (``ag_gemm`` or ``all_gather_``)."""
        T, H = out_rows.shape
        if self.world == 1:
            ops.gemm(a[:M], w, out=out_rows[:M], bias=bias)
            ops.add_rmsnorm_(out_rows, residual, norm_w, eps)
            return
        if not self.fused_gemm_available(out_rows):
            ops.gemm(a[:M], w, out=out_rows[:M], bias=bias if self.tp.rank == 0 else None)
            if self.in_kernel:
                self.fused_allreduce_add_rmsnorm_(out_rows, residual, norm_w, eps, max_ctas=max(comm_ctas, 8), mode=1)
            else:
                dist.all_reduce(out_rows, group=self.tp.group)
                ops.add_rmsnorm_(out_rows, residual, norm_w, eps)
            return
        rpr = T // self.world
        shard_res = residual[self.tp.rank * rpr:(self.tp.rank + 1) * rpr]
        _native.call("tw_gemm_rs_norm", a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), M, H, a.shape[1],
                     None if (bias is None or self.tp.rank != 0) else bias.data_ptr(), out_rows.data_ptr(), self._mc(),
                     self.buf.peer_ptrs_dev, self._flag_table(region, "tile"), self.tp.rank, self.world,
                     self.budget_ns, ops.status_word(a.device).data_ptr(), self.buf.byte_offset(out_rows), T,
                     shard_res.data_ptr(), shard_res.stride(0), norm_w.data_ptr(), eps, comm_ctas, max_ctas,
                     torch.cuda.current_stream().cuda_stream)

    def ag_gemm(self, in_rows: torch.Tensor, w: torch.Tensor, out: torch.Tensor, M: int, swiglu: bool = False,
                bias: Optional[torch.Tensor] = None, comm_ctas: int = 8, region: int = 0, max_ctas: int = 0,
                gathered: bool = False) -> torch.Tensor:
        """All-gather of ``in_rows`` (each rank holds its own shard of the [T, H] rows) fused with
        ``out[:M] = in_rows[:M] @ w.T`` (optionally SwiGLU / bias). With ``gathered=True`` the rows are
        already complete on every rank and only the GEMM runs."""
        T, H = in_rows.shape
        if gathered or self.world == 1 or not self.in_kernel:
            return ops.gemm(in_rows[:M], w, out=out[:M], bias=bias, swiglu=swiglu, max_ctas=max_ctas)
        if not self.fused_gemm_available(in_rows):
            self.all_gather_(in_rows, max_ctas=max(comm_ctas, 8))
            return ops.gemm(in_rows[:M], w, out=out[:M], bias=bias, swiglu=swiglu, max_ctas=max_ctas)
        rows_b = w.shape[0]
        N = rows_b // 2 if swiglu else rows_b
        _native.call("tw_ag_gemm", in_rows.data_ptr(), w.data_ptr(), w.stride(0), rows_b, out.data_ptr(), out.stride(0),
                     None if bias is None else bias.data_ptr(), M, N, H, int(swiglu), N if swiglu else 0, self._mc(),
                     self.buf.peer_ptrs_dev, self._flag_table(region, "shard"), self._epochs[2 * region:].data_ptr(),
                     self.tp.rank, self.world, self.budget_ns, ops.status_word(in_rows.device).data_ptr(),
                     self.buf.byte_offset(in_rows), T, comm_ctas, max_ctas, torch.cuda.current_stream().cuda_stream)
        return out[:M]
