"""Decoder-only transformer shared by the Llama, Qwen2 and Mixtral families.

Counterparts: vllm/model_executor/models/llama.py:99-590, qwen2.py, mixtral.py (with the TokenWeave
edits). Differences by design:

* the residual stream lives in one symmetric staging buffer ``[max_tokens + 512, H]`` per rank that
  o_proj / down_proj / the MoE write their partial sums into and the fused collective reduces and
  normalises in place (same aliasing as llama.py:537,568);
* the gate_up projection and SwiGLU are one GEMM (epilogue), RoPE and the KV-cache write one kernel;
* every activation workspace is allocated once for ``max_tokens`` (no allocator traffic in a step, so a
  step can be captured in a CUDA graph);
* the embedding table is replicated (see layers/embedding.py) unless ``embedding_parallel`` is set.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Optional

import torch
from torch import nn

from .. import ops
from ..config import ModelConfig
from ..layers.attention import Attention, AttentionMetadata
from ..layers.embedding import ParallelLMHead, VocabEmbedding
from ..layers.linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
from ..layers.moe import FusedMoE
from ..ops import reference
from ..parallel.comm import TPCommunicator
from ..parallel.state import get_tp, recv_from_prev_stage, send_to_next_stage
from ..parallel.symm_mem import SymmetricBuffer, create_symmetric_buffer
from ..tokenweave import schedule
from ..tokenweave.config import SplitPlan

STAGING_EXTRA_ROWS = 512   # room for the 256-row padding plus a split offset (llama.py:437 uses +512)


@dataclass
class StepInput:
    """Everything one forward pass needs besides the weights."""
    input_ids: torch.Tensor                   # [T] int32
    plan: SplitPlan
    meta: Optional[AttentionMetadata] = None  # unsplit batch
    meta0: Optional[AttentionMetadata] = None  # token subset 0 / 1 of the overlap schedule
    meta1: Optional[AttentionMetadata] = None
    logits_indices: Optional[torch.Tensor] = None   # rows whose logits are needed (last token of each request)


class Runtime:
    """Per-rank buffers and streams shared by all layers."""

    def __init__(self, cfg: ModelConfig, max_tokens: int, device: torch.device, tw_cfg, provider: Optional[str] = None):
        tp = get_tp()
        self.device = device
        self.max_tokens = max_tokens
        rows = max_tokens + STAGING_EXTRA_ROWS
        H, D = cfg.hidden_size, cfg.head_dim
        dt = cfg.dtype
        hq = cfg.num_q_heads // tp.world_size
        hkv = max(1, cfg.num_kv_heads // tp.world_size)
        allow_mc = tw_cfg.transport in ("auto", "multimem")
        self.staging: SymmetricBuffer = create_symmetric_buffer(rows, H, dt, tp, provider, allow_mc)
        self.hidden = self.staging.tensor
        self.residual = torch.zeros(rows, H, dtype=dt, device=device)
        self.qkv = torch.zeros(rows, (hq + 2 * hkv) * D, dtype=dt, device=device)
        self.attn_out = torch.zeros(rows, hq * D, dtype=dt, device=device)
        inter = cfg.intermediate_size // tp.world_size
        self.act = None if cfg.is_moe else torch.zeros(rows, inter, dtype=dt, device=device)
        self.comm = TPCommunicator(self.staging, tp, tw_cfg.wait_budget_ms, tw_cfg.transport)
        self.flag_buf = None
        if self.comm.in_kernel:
            # tile counters and shard epochs of the GEMM kernels that are fused with their collectives
            self.flag_buf = create_symmetric_buffer(1, 8192, dt, tp, provider, allow_multicast=False)
            self.comm.attach_flag_buffer(self.flag_buf)
        if device.type == "cuda":
            self.comm_stream = torch.cuda.Stream(device=device, priority=-1)
            self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        else:
            self.comm_stream = None
            self.sm_count = 0
        self.cos_sin = reference.build_cos_sin_cache(D, cfg.max_model_len, cfg.rope_theta, cfg.rope_scaling, device)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, *, device):
        super().__init__()
        tp = get_tp()
        dt = cfg.dtype
        H, D = cfg.hidden_size, cfg.head_dim
        self.qkv_proj = QKVParallelLinear(H, D, cfg.num_q_heads, cfg.num_kv_heads, cfg.qkv_bias, dtype=dt, device=device)
        self.o_proj = RowParallelLinear(cfg.num_q_heads * D, H, False, dtype=dt, device=device)
        self.attn = Attention(self.qkv_proj.q_heads, self.qkv_proj.kv_heads, D, sliding_window=cfg.sliding_window,
                              logit_softcap=cfg.attn_logit_softcapping)
        if cfg.qk_norm:
            # one weight vector per projection, shared by all heads (and therefore by all ranks)
            self.q_norm_w = nn.Parameter(torch.ones(D, dtype=dt, device=device), requires_grad=False)
            self.k_norm_w = nn.Parameter(torch.ones(D, dtype=dt, device=device), requires_grad=False)
            self.attn.qk_norm = (self.q_norm_w, self.k_norm_w, cfg.rms_norm_eps)
        self.input_norm_w = nn.Parameter(torch.ones(H, dtype=dt, device=device), requires_grad=False)
        self.post_norm_w = nn.Parameter(torch.ones(H, dtype=dt, device=device), requires_grad=False)
        if cfg.is_moe:
            self.moe = FusedMoE(cfg.num_experts, cfg.num_experts_per_tok, H, cfg.intermediate_size, dtype=dt, device=device,
                                expert_parallel=cfg.expert_parallel)
            self.gate_up_proj = self.down_proj = None
        else:
            self.moe = None
            self.gate_up_proj = MergedColumnParallelLinear(H, [cfg.intermediate_size] * 2, False, dtype=dt, device=device)
            self.down_proj = RowParallelLinear(cfg.intermediate_size, H, False, dtype=dt, device=device)

    layer_idx = 0        # set by the model; keys the LoRA weights of this layer

    def _lora_segments(self, rows: torch.Tensor, n: int, rt: Runtime) -> list:
        """Adapters used by the token rows of this block call (``rows`` is a view of the staging buffer, so
        its offset tells which rows of the step it covers)."""
        lora = getattr(rt, "lora", None)
        if lora is None or not lora.active:
            return []
        row0 = (rows.data_ptr() - rt.hidden.data_ptr()) // (rt.hidden.stride(0) * rt.hidden.element_size())
        return lora.segments(int(row0), n, rows.device)

    def attn_block(self, rows: torch.Tensor, n: int, meta: AttentionMetadata, rt: Runtime, max_ctas: int) -> None:
        """rows[:n] (normalised activations) -> this rank's partial o_proj output, in place."""
        if n == 0:
            return
        segs = self._lora_segments(rows, n, rt)
        qkv = self.qkv_proj(rows[:n], out=rt.qkv[:n], max_ctas=max_ctas)
        if segs:
            from ..lora import LoRAManager
            LoRAManager.apply(segs, self.layer_idx, "qkv_proj", rows[:n], qkv)
        attn_out = self.attn(qkv, rt.cos_sin, meta, rt.attn_out[:n], max_ctas=max_ctas)
        if segs:
            # the o_proj output overwrites rows[:n], which is also nothing the delta needs: the delta reads attn_out
            self.o_proj(attn_out, out=rows[:n], max_ctas=max_ctas)
            LoRAManager.apply(segs, self.layer_idx, "o_proj", attn_out, rows[:n])
            return
        self.o_proj(attn_out, out=rows[:n], max_ctas=max_ctas)

    # ---- the same blocks with every GEMM fused with its neighbouring collective ----
    def attn_block_fused(self, rows: torch.Tensor, n: int, meta: AttentionMetadata, rt: Runtime, comm, residual,
                         eps: float, comm_ctas: int, gathered: bool) -> None:
        """rows: [T_pad, H]; on entry this rank's shard holds the normalised input (all rows if ``gathered``);
        on exit this rank's shard holds the post-attention-norm output and its residual shard is updated."""
        qkv = comm.ag_gemm(rows, self.qkv_proj.weight, rt.qkv, n, bias=self.qkv_proj.bias, comm_ctas=comm_ctas,
                           gathered=gathered)
        attn_out = self.attn(qkv, rt.cos_sin, meta, rt.attn_out[:n])
        comm.gemm_rs_norm_(attn_out, self.o_proj.weight, rows, n, residual, self.post_norm_w, eps, comm_ctas)

    def mlp_block_fused(self, rows: torch.Tensor, n: int, rt: Runtime, comm, residual, next_norm_w, eps: float,
                        comm_ctas: int) -> None:
        act = comm.ag_gemm(rows, self.gate_up_proj.weight, rt.act, n, swiglu=True, comm_ctas=comm_ctas)
        comm.gemm_rs_norm_(act, self.down_proj.weight, rows, n, residual, next_norm_w, eps, comm_ctas)

    def mlp_block(self, rows: torch.Tensor, n: int, rt: Runtime, max_ctas: int) -> None:
        if n == 0:
            return
        if self.moe is not None:
            self.moe(rows[:n], out=rows[:n], max_ctas=max_ctas)
            return
        segs = self._lora_segments(rows, n, rt)
        if segs:
            # the adapter's gate / up deltas go in before the activation, so the SwiGLU epilogue cannot be used
            from ..lora import LoRAManager
            gate_up = self.gate_up_proj(rows[:n], max_ctas=max_ctas)
            LoRAManager.apply(segs, self.layer_idx, "gate_up_proj", rows[:n], gate_up)
            act = ops.swiglu(gate_up, out=rt.act[:n])
            self.down_proj(act, out=rows[:n], max_ctas=max_ctas)
            LoRAManager.apply(segs, self.layer_idx, "down_proj", act, rows[:n])
            return
        act = self.gate_up_proj.forward_swiglu(rows[:n], out=rt.act[:n], max_ctas=max_ctas)
        self.down_proj(act, out=rows[:n], max_ctas=max_ctas)


class DecoderModel(nn.Module):
    architecture = "llama"

    def __init__(self, cfg: ModelConfig, *, device, embedding_parallel: bool = False):
        super().__init__()
        self.cfg = cfg
        dt = cfg.dtype
        self.embed_tokens = VocabEmbedding(cfg.vocab_size, cfg.hidden_size, embedding_parallel, dtype=dt, device=device)
        # pipeline parallelism: this process holds a consecutive range of the layers (all of them at one stage;
        # early stages take the remainder, vllm/distributed/utils.py ``get_pp_indices``)
        tp = get_tp()
        per, extra = divmod(cfg.num_layers, tp.pp_size)
        self.first_layer = tp.pp_rank * per + min(tp.pp_rank, extra)
        self.end_layer = self.first_layer + per + (1 if tp.pp_rank < extra else 0)
        if self.end_layer == self.first_layer:
            raise ValueError(f"{cfg.num_layers} layers cannot fill {tp.pp_size} pipeline stages")
        self.layers = nn.ModuleList([DecoderLayer(cfg, device=device) for _ in range(self.first_layer, self.end_layer)])
        for i, layer in enumerate(self.layers):
            layer.layer_idx = self.first_layer + i
        self.norm_w = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dt, device=device), requires_grad=False)
        # A stage that is not the last closes its last layer with the NEXT stage's first input norm (the fused
        # collective applies the following block's norm), so it keeps a copy of that weight.
        self.boundary_norm_w = None
        if not tp.is_last_stage:
            self.boundary_norm_w = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dt, device=device), requires_grad=False)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, dtype=dt, device=device)
        self.rt: Optional[Runtime] = None
        self.tw_mode = "overlap"

    # ---- runtime -------------------------------------------------------------------------
    def setup_runtime(self, max_tokens: int, tw_cfg, provider: Optional[str] = None,
                      disable_custom_all_reduce: bool = True) -> Runtime:
        device = self.norm_w.device
        self.rt = Runtime(self.cfg, max_tokens, device, tw_cfg, provider)
        self.tw_mode = tw_cfg.mode
        # library baselines: NCCL through the package's own communicator (graph-capturable, on the current
        # stream) for "baseline_nccl" and the logits gather; peer-to-peer all-reduce when the engine allows it
        from .. import envs
        if envs.TW_USE_PYNCCL and self.rt.comm.enable_pynccl():
            self.lm_head.comm = self.rt.comm
        if not disable_custom_all_reduce:
            self.rt.comm.enable_custom_all_reduce()
        return self.rt

    def kv_cache_bytes_per_block(self, block_size: int) -> int:
        l0 = self.layers[0]
        return 2 * block_size * l0.attn.hkv * l0.attn.head_dim * self.cfg.dtype.itemsize * len(self.layers)

    def init_kv_cache(self, num_blocks: int, block_size: int) -> None:
        dev = self.norm_w.device
        for layer in self.layers:
            a = layer.attn
            k = torch.zeros(num_blocks, block_size, a.hkv, a.head_dim, dtype=self.cfg.dtype, device=dev)
            v = torch.zeros_like(k)
            a.bind_kv_cache(k, v)

    # ---- forward -------------------------------------------------------------------------
    @torch.inference_mode()
    def forward(self, step: StepInput) -> torch.Tensor:
        """Runs the decoder stack; returns the final-norm hidden rows ``[T, H]`` (a view of the staging buffer)."""
        rt, plan, cfg = self.rt, step.plan, self.cfg
        T, Tp = plan.num_tokens, plan.padded_tokens
        assert Tp <= rt.hidden.shape[0], "step exceeds the staging buffer"
        hidden, residual = rt.hidden, rt.residual
        eps = cfg.rms_norm_eps
        stage = get_tp()
        if stage.is_first_stage:
            if Tp > T:
                hidden[T:Tp].zero_()
            self.embed_tokens(step.input_ids, out=hidden[:T])
            pending = self.embed_tokens.parallel and self.tw_mode not in ("no_ar", "no_ar_no_ln")
            if pending:
                residual[:Tp].zero_()
            else:
                if Tp > T:
                    residual[T:Tp].zero_()
                ops.rmsnorm_copy_(hidden[:T], residual[:T], self.layers[0].input_norm_w, eps)
        else:
            # the previous stage left the normalised input of our first layer and the residual stream (whatever
            # its layout across the tensor-parallel ranks: the peer with the same TP rank holds the same rows)
            recv_from_prev_stage(hidden[:Tp], residual[:Tp])
            pending = False
        close_w = self.norm_w if stage.is_last_stage else self.boundary_norm_w
        if plan.overlap:
            schedule.run_overlap(self.layers, close_w, hidden, residual, step.meta0, step.meta1, plan, rt.comm,
                                 rt, eps, pending)
        elif self.tw_mode == "fused_gemm":
            schedule.run_fused_gemm(self.layers, close_w, hidden, residual, step.meta, plan, rt.comm, rt, eps,
                                    pending)
        elif self.tw_mode in ("overlap", "fuse_only"):
            schedule.run_fuse_only(self.layers, close_w, hidden, residual, step.meta, plan, rt.comm, rt, eps,
                                   pending)
        else:
            schedule.run_baseline(self.layers, close_w, hidden, residual, step.meta, plan, rt.comm, rt, eps,
                                  self.tw_mode, pending)
        if not stage.is_last_stage:
            send_to_next_stage(hidden[:Tp], residual[:Tp])
        return hidden[:T]

    @torch.inference_mode()
    def compute_logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        return self.lm_head(hidden_rows)

    # ---- weights -------------------------------------------------------------------------
    def init_dummy_weights(self, seed: int = 0) -> None:
        """Random weights of the checkpoint's statistics (the reference's DummyModelLoader,
        vllm/model_executor/model_loader/loader.py:476-500). Every rank draws the full-size tensor
        stream from the same seed and keeps its shard, so TP runs are comparable across sizes only
        statistically; for exact TP-vs-single comparisons load a checkpoint instead."""
        std = self.cfg.init_std
        gen_dev = self.norm_w.device
        g = torch.Generator(device=gen_dev)
        g.manual_seed(seed + 1234567 * (get_tp().rank + 1))
        for name, p in self.named_parameters():
            if name.endswith("norm_w"):
                p.data.fill_(1.0)
            elif p.dim() == 1:
                p.data.zero_()
            else:
                p.data.normal_(0.0, std, generator=g)
        if self.embed_tokens.parallel is False and get_tp().world_size > 1:
            # a replicated table must be identical on all ranks
            g2 = torch.Generator(device=gen_dev)
            g2.manual_seed(seed + 99)
            self.embed_tokens.weight.data.normal_(0.0, std, generator=g2)
        if get_tp().world_size > 1:
            for layer in self.layers:
                if layer.moe is not None:
                    g3 = torch.Generator(device=gen_dev)
                    g3.manual_seed(seed + 7)
                    layer.moe.gate.data.normal_(0.0, std, generator=g3)

    # HuggingFace name -> (module path, shard id)
    STACKED = [(".q_proj", ".qkv_proj", "q"), (".k_proj", ".qkv_proj", "k"), (".v_proj", ".qkv_proj", "v"),
               (".gate_proj", ".gate_up_proj", 0), (".up_proj", ".gate_up_proj", 1)]
    # HuggingFace name of an already fused projection -> (module, shard ids, rows of each piece)
    PACKED = {
        ".qkv_proj": lambda c: ("qkv_proj", ("q", "k", "v"),
                                [c.num_q_heads * c.head_dim, c.num_kv_heads * c.head_dim, c.num_kv_heads * c.head_dim]),
        ".gate_up_proj": lambda c: ("gate_up_proj", (0, 1), [c.intermediate_size, c.intermediate_size]),
    }

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        """Load HuggingFace-layout tensors (``model.layers.N.self_attn.q_proj.weight`` ...), sharding on
        the fly. Returns the names that were consumed."""
        loaded: set[str] = set()
        saw_lm_head = False
        for name, tensor in weights:
            if "rotary_emb.inv_freq" in name:
                continue
            n = name[len("model."):] if name.startswith("model.") else name
            if n == "embed_tokens.weight":
                self.embed_tokens.weight_loader(self.embed_tokens.weight, tensor)
                if self.cfg.tie_word_embeddings:
                    self.lm_head.weight_loader(self.lm_head.weight, tensor)
            elif n == "norm.weight":
                self.norm_w.data.copy_(tensor)
            elif n == "lm_head.weight":
                saw_lm_head = True
                self.lm_head.weight_loader(self.lm_head.weight, tensor)
            elif n.startswith("layers."):
                _, idx, rest = n.split(".", 2)
                li = int(idx)
                if li == self.end_layer and self.boundary_norm_w is not None and rest == "input_layernorm.weight":
                    self.boundary_norm_w.data.copy_(tensor)       # the next stage's first input norm
                    loaded.add(name)
                    continue
                if not self.first_layer <= li < self.end_layer:
                    continue
                self._load_layer_weight(self.layers[li - self.first_layer], rest, tensor)
            else:
                continue
            loaded.add(name)
        return loaded

    def _load_layer_weight(self, layer: DecoderLayer, rest: str, t: torch.Tensor) -> None:
        if rest == "input_layernorm.weight":
            layer.input_norm_w.data.copy_(t)
            return
        if rest == "post_attention_layernorm.weight":
            layer.post_norm_w.data.copy_(t)
            return
        if rest.startswith("block_sparse_moe."):
            sub = rest[len("block_sparse_moe."):]
            if sub == "gate.weight":
                layer.moe.gate.data.copy_(t)
            else:                                   # experts.{e}.w{1,2,3}.weight
                _, e, which, _ = sub.split(".")
                layer.moe.load_expert_weight(int(e), which, t)
            return
        rest = rest.replace("self_attn.", "").replace("mlp.", "")
        if rest in ("q_norm.weight", "k_norm.weight"):
            getattr(layer, rest[0] + "_norm_w").data.copy_(t)
            return
        kind = "bias" if rest.endswith(".bias") else "weight"
        stem = "." + rest[: -len(kind) - 1]
        if stem in self.PACKED:
            # checkpoints that store the fused projection (Phi-3): cut it at the full-model boundaries and
            # hand the pieces to the same shard loaders as separate tensors would get
            ours, shards, sizes = self.PACKED[stem](self.cfg)
            mod = getattr(layer, ours)
            for shard, piece in zip(shards, t.split(sizes, dim=0)):
                mod.weight_loader(getattr(mod, kind), piece, shard)
            return
        for hf, ours, shard in self.STACKED:
            if stem == hf:
                mod = getattr(layer, ours[1:])
                mod.weight_loader(getattr(mod, kind), t, shard)
                return
        mod = getattr(layer, stem[1:])
        mod.weight_loader(getattr(mod, kind), t)
