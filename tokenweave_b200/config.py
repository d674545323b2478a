"""Configuration dataclasses and the flag system.

Three tiers, as in the reference (vllm/config.py:201-3619, vllm/engine/arg_utils.py, vllm/envs.py):
``EngineArgs`` (constructor / CLI flags) folds into ``EngineConfig`` (model, cache, parallel,
scheduler and TokenWeave sections); environment variables ``TW_*`` are read lazily through
:mod:`tokenweave_b200.envs`; per-model TokenWeave JSON files map a token count to a split point and
communication-SM budget (:mod:`tokenweave_b200.tokenweave.config`).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "float16": torch.float16, "half": torch.float16, "auto": None}


@dataclass
class ModelConfig:
    """Architecture of a decoder-only transformer (Llama-3.x, Qwen2.5, Mixtral layouts)."""
    name: str = "tiny-llama"
    architecture: str = "llama"          # "llama" | "qwen2" | "mixtral" | "qwen3" | "mistral" | "phi3"
    hidden_size: int = 256
    num_layers: int = 2
    num_q_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 688
    vocab_size: int = 1024
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: Optional[dict] = None
    qkv_bias: bool = False
    qk_norm: bool = False                # RMSNorm over head_dim on every q and k head before rope (Qwen3)
    sliding_window: int = 0              # a query sees the last N keys only (Mistral-7B v0.1: 4096); 0 = full attention
    attn_logit_softcapping: float = 0.0  # attention scores pass through cap * tanh(s / cap) (Gemma-2 style); 0 = off
    num_experts: int = 0                 # 0 = dense MLP
    num_experts_per_tok: int = 2
    max_model_len: int = 8192
    tie_word_embeddings: bool = False
    dtype: torch.dtype = torch.bfloat16
    eos_token_id: Optional[int] = None
    expert_parallel: bool = False       # MoE: whole experts per rank instead of tensor-sharded experts
    init_std: float = 0.02
    path: Optional[str] = None           # checkpoint directory (None: random init)
    checkpoint_quantization: Optional[str] = None    # "fp8" when the checkpoint's config says its weights are fp8
    # weight-only integer checkpoints (AWQ, GPTQ): {"method", "bits", "group_size", "zeros_plus_one"}; their packed
    # tensors are expanded to the model's dtype while loading (models/loader.py)
    checkpoint_packing: Optional[dict] = None

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def num_params(self) -> int:
        h, l = self.hidden_size, self.num_layers
        attn = h * (self.num_q_heads + 2 * self.num_kv_heads) * self.head_dim + self.num_q_heads * self.head_dim * h
        mlp = 3 * h * self.intermediate_size * max(1, self.num_experts)
        emb = self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return l * (attn + mlp + 2 * h) + emb + h

    @staticmethod
    def from_hf_dict(cfg: dict, name: str = "", path: Optional[str] = None) -> "ModelConfig":
        archs = cfg.get("architectures") or [cfg.get("model_type", "llama")]
        a = archs[0].lower()
        if any(k in a for k in ("moe", "vl", "omni", "audio")) and "mixtral" not in a:
            raise ValueError(f"unsupported architecture {archs[0]!r}")
        arch = ("mixtral" if "mixtral" in a else "qwen3" if "qwen3" in a else "qwen2" if "qwen2" in a
                else "phi3" if "phi3" in a else "mistral" if "mistral" in a else "llama")
        heads = cfg["num_attention_heads"]
        head_dim = cfg.get("head_dim") or cfg["hidden_size"] // heads
        dt = _DTYPES.get(str(cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))), torch.bfloat16) or torch.bfloat16
        eos = cfg.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0]
        # newer Hugging Face configs keep theta and the scaling rule together under "rope_parameters"
        rp = dict(cfg.get("rope_parameters") or {})
        if rp:
            cfg = dict(cfg)
            cfg.setdefault("rope_theta", rp.pop("rope_theta", None) or (1e6 if arch != "llama" else 10000.0))
            if rp.get("rope_type", "default") != "default":
                cfg.setdefault("rope_scaling", rp)
        max_len = cfg.get("max_position_embeddings", 8192)
        window = cfg.get("sliding_window")
        window = int(window) if window and cfg.get("use_sliding_window", True) and window < max_len else 0
        return ModelConfig(
            name=name or cfg.get("_name_or_path", arch), architecture=arch, hidden_size=cfg["hidden_size"],
            num_layers=cfg["num_hidden_layers"], num_q_heads=heads,
            num_kv_heads=cfg.get("num_key_value_heads", heads), head_dim=head_dim,
            intermediate_size=cfg["intermediate_size"], vocab_size=cfg["vocab_size"],
            rms_norm_eps=cfg.get("rms_norm_eps", 1e-6 if arch in ("qwen2", "qwen3") else 1e-5),
            rope_theta=cfg.get("rope_theta") or (1e6 if arch in ("qwen2", "qwen3", "mixtral") else 10000.0),
            rope_scaling=cfg.get("rope_scaling"), qkv_bias=cfg.get("attention_bias", arch == "qwen2"),
            qk_norm=arch == "qwen3", sliding_window=window,
            attn_logit_softcapping=float(cfg.get("attn_logit_softcapping") or 0.0),
            num_experts=cfg.get("num_local_experts", 0), num_experts_per_tok=cfg.get("num_experts_per_tok", 2),
            max_model_len=max_len,
            tie_word_embeddings=cfg.get("tie_word_embeddings", False), dtype=dt, eos_token_id=eos, path=path,
            checkpoint_quantization=ModelConfig._quant_of(cfg), checkpoint_packing=ModelConfig._packing_of(cfg))

    @staticmethod
    def _quant_of(cfg: dict) -> Optional[str]:
        """"fp8" for checkpoints quantised to fp8 (``quant_method`` fp8, or compressed-tensors with 8-bit float
        weights); other schemes are not served."""
        qc = cfg.get("quantization_config") or {}
        method = str(qc.get("quant_method", "")).lower()
        if not method:
            return None
        if method == "fp8":
            return "fp8"
        if method in ("awq", "gptq"):
            return None                  # weight-only integers: expanded at load time, see _packing_of
        if method == "compressed-tensors":
            groups = (qc.get("config_groups") or {}).values()
            if groups and all((g.get("weights") or {}).get("type") == "float" and (g.get("weights") or {}).get("num_bits") == 8
                              for g in groups):
                return "fp8"
        raise ValueError(f"checkpoint quantised with {method!r}: fp8, AWQ and GPTQ checkpoints are served")

    @staticmethod
    def _packing_of(cfg: dict) -> Optional[dict]:
        """Packing of a weight-only integer checkpoint: AWQ (``quant_method`` awq, ``version`` gemm, 4 bits, the
        layout vllm/model_executor/layers/quantization/awq.py reads) or GPTQ (4 or 8 bits, with or without
        activation order, vllm/model_executor/layers/quantization/gptq.py)."""
        qc = cfg.get("quantization_config") or {}
        method = str(qc.get("quant_method", "")).lower()
        if method not in ("awq", "gptq"):
            return None
        bits = int(qc.get("bits", qc.get("w_bit", 4)))
        group = int(qc.get("group_size", qc.get("q_group_size", 128)))
        if method == "awq":
            if bits != 4 or str(qc.get("version", "gemm")).lower() != "gemm":
                raise ValueError("AWQ checkpoints are served in the 4-bit GEMM layout only")
            return {"method": "awq", "bits": 4, "group_size": group, "zeros_plus_one": False}
        if bits not in (4, 8):
            raise ValueError(f"GPTQ checkpoints are served with 4 or 8 bits (got {bits})")
        # the first GPTQ format stores zero points minus one; "gptq_v2" stores them as they are
        v2 = str(qc.get("checkpoint_format", "gptq")).lower() == "gptq_v2"
        return {"method": "gptq", "bits": bits, "group_size": group, "zeros_plus_one": not v2}

    @staticmethod
    def from_pretrained(path: str) -> "ModelConfig":
        p = Path(path)
        with open(p / "config.json") as f:
            return ModelConfig.from_hf_dict(json.load(f), name=p.name, path=str(p))


def _preset(**kw) -> ModelConfig:
    return ModelConfig(**kw)


MODEL_PRESETS: dict[str, dict[str, Any]] = {
    # correctness configuration: fp32 on CPU, split path must equal the unsplit path
    "tiny-llama": dict(architecture="llama", hidden_size=256, num_layers=2, num_q_heads=4, num_kv_heads=2,
                       head_dim=64, intermediate_size=688, vocab_size=1024, rms_norm_eps=1e-5,
                       rope_theta=500000.0, max_model_len=2048),
    "tiny-llama-d128": dict(architecture="llama", hidden_size=512, num_layers=2, num_q_heads=4, num_kv_heads=2,
                            head_dim=128, intermediate_size=1024, vocab_size=2048, rms_norm_eps=1e-5,
                            rope_theta=500000.0, max_model_len=4096),
    # eight query heads: shards over 8 tensor-parallel ranks (the two KV heads are then replicated four times)
    "tiny-llama-h8": dict(architecture="llama", hidden_size=1024, num_layers=2, num_q_heads=8, num_kv_heads=2,
                          head_dim=128, intermediate_size=2048, vocab_size=2048, rms_norm_eps=1e-5,
                          rope_theta=500000.0, max_model_len=4096),
    "tiny-qwen2": dict(architecture="qwen2", hidden_size=512, num_layers=2, num_q_heads=4, num_kv_heads=2,
                       head_dim=128, intermediate_size=1024, vocab_size=2048, rms_norm_eps=1e-6,
                       rope_theta=1e6, qkv_bias=True, max_model_len=4096),
    "tiny-mixtral": dict(architecture="mixtral", hidden_size=512, num_layers=2, num_q_heads=4, num_kv_heads=2,
                         head_dim=128, intermediate_size=512, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=1e6,
                         num_experts=8, num_experts_per_tok=2, max_model_len=4096),
    "tiny-qwen3": dict(architecture="qwen3", hidden_size=512, num_layers=2, num_q_heads=4, num_kv_heads=2,
                       head_dim=128, intermediate_size=1024, vocab_size=2048, rms_norm_eps=1e-6,
                       rope_theta=1e6, qk_norm=True, max_model_len=4096),
    "qwen3-32b": dict(architecture="qwen3", hidden_size=5120, num_layers=64, num_q_heads=64, num_kv_heads=8,
                      head_dim=128, intermediate_size=25600, vocab_size=151936, rms_norm_eps=1e-6,
                      rope_theta=1e6, qk_norm=True, max_model_len=40960),
    "mistral-large-2": dict(architecture="mistral", hidden_size=12288, num_layers=88, num_q_heads=96, num_kv_heads=8,
                            head_dim=128, intermediate_size=28672, vocab_size=32768, rms_norm_eps=1e-5,
                            rope_theta=1e6, max_model_len=131072),
    "phi-3-medium-4k": dict(architecture="phi3", hidden_size=5120, num_layers=40, num_q_heads=40, num_kv_heads=10,
                            head_dim=128, intermediate_size=17920, vocab_size=32064, rms_norm_eps=1e-5,
                            rope_theta=10000.0, max_model_len=4096),
    "llama-3.3-70b": dict(architecture="llama", hidden_size=8192, num_layers=80, num_q_heads=64, num_kv_heads=8,
                          head_dim=128, intermediate_size=28672, vocab_size=128256, rms_norm_eps=1e-5,
                          rope_theta=500000.0, max_model_len=131072,
                          rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                            high_freq_factor=4.0, original_max_position_embeddings=8192)),
    "llama-3.1-8b": dict(architecture="llama", hidden_size=4096, num_layers=32, num_q_heads=32, num_kv_heads=8,
                         head_dim=128, intermediate_size=14336, vocab_size=128256, rms_norm_eps=1e-5,
                         rope_theta=500000.0, max_model_len=131072,
                         rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                           high_freq_factor=4.0, original_max_position_embeddings=8192)),
    "qwen2.5-72b": dict(architecture="qwen2", hidden_size=8192, num_layers=80, num_q_heads=64, num_kv_heads=8,
                        head_dim=128, intermediate_size=29568, vocab_size=152064, rms_norm_eps=1e-6,
                        rope_theta=1e6, qkv_bias=True, max_model_len=32768),
    "mixtral-8x22b": dict(architecture="mixtral", hidden_size=6144, num_layers=56, num_q_heads=48, num_kv_heads=8,
                          head_dim=128, intermediate_size=16384, vocab_size=32768, rms_norm_eps=1e-5,
                          rope_theta=1e6, num_experts=8, num_experts_per_tok=2, max_model_len=65536),
}
_ALIASES = {"meta-llama/llama-3.3-70b-instruct": "llama-3.3-70b", "qwen/qwen2.5-72b-instruct": "qwen2.5-72b",
            "mistralai/mixtral-8x22b-instruct-v0.1": "mixtral-8x22b", "meta-llama/llama-3.1-8b-instruct": "llama-3.1-8b"}


def resolve_model_config(model: "str | ModelConfig", dtype: Optional[str] = None,
                         max_model_len: Optional[int] = None, num_layers: Optional[int] = None) -> ModelConfig:
    """A preset name, a HuggingFace-style name of a supported model, or a checkpoint directory."""
    if isinstance(model, ModelConfig):
        cfg = dataclasses.replace(model)
    else:
        key = _ALIASES.get(model.lower(), model.lower())
        if key in MODEL_PRESETS:
            cfg = ModelConfig(name=key, **MODEL_PRESETS[key])
        elif Path(model).is_dir() and (Path(model) / "config.json").exists():
            cfg = ModelConfig.from_pretrained(model)
        else:
            raise ValueError(f"unknown model {model!r}: not a preset ({sorted(MODEL_PRESETS)}) nor a checkpoint directory")
    if dtype and _DTYPES.get(dtype) is not None:
        cfg.dtype = _DTYPES[dtype]
    if max_model_len:
        cfg.max_model_len = max_model_len
    if num_layers:
        cfg.num_layers = num_layers
    return cfg


@dataclass
class CacheConfig:
    block_size: int = 128                 # tokens per KV page (TMA-friendly; the reference uses 16)
    gpu_memory_utilization: float = 0.90
    num_gpu_blocks: Optional[int] = None  # override the profiled value
    enable_prefix_caching: bool = False


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    # "uni": in-process worker; "mp": one spawned worker process per GPU;
    # "external_launcher": this process is one rank of a torchrun job (SPMD, deterministic scheduling)
    distributed_executor_backend: str = "auto"
    disable_custom_all_reduce: bool = True
    nvls: bool = True                     # allow multimem transport when the hardware offers it
    # data parallelism: independent engine replicas, each a TP group on its own GPUs
    # (replica r uses devices [r * tp, (r + 1) * tp))
    data_parallel_size: int = 1
    data_parallel_rank: int = 0
    # pipeline parallelism: the layers are cut into this many consecutive stages of tensor_parallel_size ranks
    pipeline_parallel_size: int = 1

    @property
    def world_size(self) -> int:
        """Ranks of one engine replica."""
        return self.tensor_parallel_size * self.pipeline_parallel_size

    @property
    def device_offset(self) -> int:
        return self.data_parallel_rank * self.world_size


@dataclass
class SchedulerConfig:
    max_num_batched_tokens: int = 8192
    max_num_seqs: int = 256
    enable_chunked_prefill: bool = True
    max_model_len: int = 8192
    policy: str = "fcfs"                  # "fcfs" | "priority" (lower value first, arrival order among equals)
    # > 0: a request gets at most this many new tokens per step, so that one long prompt does not take a whole
    # step's budget and shorter requests behind it start sooner (vllm/v1/core/sched/scheduler.py:181-184, 333-336)
    long_prefill_token_threshold: int = 0


@dataclass
class TokenWeaveConfig:
    """How the tensor-parallel all-reduce of every layer is executed.

    mode:
      "overlap"           token split + fused RS/add/RMSNorm/AG on a second stream (the product path)
      "fuse_only"         fused kernel, no split
      "baseline_multimem" in-kernel all-reduce, separate add+RMSNorm kernel
      "baseline_nccl"     NCCL all-reduce, separate add+RMSNorm kernel
      "baseline_custom_ar" peer-to-peer one-shot / two-shot all-reduce for messages up to 8 MB when
                          ``disable_custom_all_reduce=False`` (NCCL otherwise), separate add+RMSNorm kernel
      "no_ar"             communication deleted (numerically wrong upper bound); also the cost-attribution
                          variants "no_ar1", "no_ar2", "no_ln1", "no_ln2", "no_ar_no_ln"
    """
    mode: str = "overlap"
    config_path: Optional[str] = None     # JSON: tokens -> {attention_ctas, mlp_ctas, split_offset}
    overlap_threshold: Optional[int] = None  # tokens; None: 1024 (llama, qwen2) / 2048 (mixtral)
    fuse_only_ctas: int = 16
    transport: str = "auto"               # "auto" | "multimem" | "p2p"
    split_offset: Optional[int] = None    # overrides the file (and TW_SPLIT_OFFSET)
    attention_ctas: Optional[int] = None
    mlp_ctas: Optional[int] = None
    use_cuda_graphs: bool = False
    wait_budget_ms: int = 2000            # budget of every cross-GPU wait inside a kernel
    force_overlap: bool = False           # take the split schedule even at TP=1 (tests, ablations)


@dataclass
class EngineConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    cache: CacheConfig = field(default_factory=CacheConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    tokenweave: TokenWeaveConfig = field(default_factory=TokenWeaveConfig)
    load_format: str = "auto"             # "auto" | "dummy" | "safetensors" | "sharded_state"
    quantization: Optional[str] = None    # None | "fp8" | "int8" (8-bit weights per channel, dynamic per-token activations)
    seed: int = 0
    device: str = "auto"                  # "auto" | "cuda" | "cpu"
    enforce_eager: bool = True
    tokenizer: Optional[str] = None
    skip_tokenizer_init: bool = False
    disable_log_stats: bool = True
    enable_sleep_mode: bool = False       # weights and KV cache on the VMM allocator: LLM.sleep() frees their memory
    speculative: Any = None               # engine.spec_decode.SpecDecodeConfig (n-gram drafts for greedy requests)
    enable_lora: bool = False             # serve requests through LoRA adapters (tokenweave_b200.lora)
    max_loras: int = 8                    # adapters resident per worker (least recently used is evicted)
    kv_transfer: Any = None               # engine.kv_connector.KVTransferConfig (blocks shared through storage)
    # scheduler + executor in a process of their own behind ZMQ / msgpack (engine/core_client.py); the front end
    # (tokeniser, detokeniser, output assembly) then overlaps with scheduling and kernel launches
    engine_core_process: bool = False
    engine_core_timeout_s: float = 300.0  # a step result that takes longer than this means the core is stuck

    def resolved_device(self) -> str:
        if self.device != "auto":
            return self.device
        return "cuda" if torch.cuda.is_available() else "cpu"


@dataclass
class EngineArgs:
    """Constructor / command-line flags (subset of vllm/engine/arg_utils.py that TokenWeave runs use)."""
    model: Any = "tiny-llama"
    tokenizer: Optional[str] = None
    skip_tokenizer_init: bool = False
    dtype: str = "auto"
    seed: int = 0
    max_model_len: Optional[int] = None
    tensor_parallel_size: int = 1
    distributed_executor_backend: str = "auto"
    pipeline_parallel_size: int = 1       # pipeline stages (consecutive layer ranges), each a tensor-parallel group
    data_parallel_size: int = 1           # engine replicas behind one front end (entrypoints/api_server.py)
    data_parallel_rank: int = 0           # which replica this engine is: its GPUs start at rank * tensor_parallel_size
    block_size: int = 128
    gpu_memory_utilization: float = 0.90
    num_gpu_blocks_override: Optional[int] = None
    enable_prefix_caching: bool = False
    max_num_batched_tokens: Optional[int] = None
    max_num_seqs: int = 256
    enable_chunked_prefill: bool = True
    scheduling_policy: str = "fcfs"       # "fcfs" | "priority": requests carry a priority, lower values run first
    long_prefill_token_threshold: int = 0     # > 0: cap on the new tokens of one request per step
    enforce_eager: bool = True
    enable_expert_parallel: bool = False
    disable_custom_all_reduce: bool = True
    load_format: str = "auto"
    quantization: Optional[str] = None
    device: str = "auto"
    num_hidden_layers_override: Optional[int] = None
    disable_log_stats: bool = True
    enable_sleep_mode: bool = False       # weights and KV cache on the VMM allocator: LLM.sleep() frees their memory
    # {"method": "ngram", "num_speculative_tokens": k, "prompt_lookup_max": n, "prompt_lookup_min": m}, or just k
    speculative_config: Any = None
    # {"kv_connector": "SharedStorageConnector", "kv_role": "kv_producer" | "kv_consumer" | "kv_both",
    #  "kv_connector_extra_config": {"shared_storage_path": dir}}: KV blocks published to / fetched from storage
    kv_transfer_config: Any = None
    engine_core_process: bool = False     # run scheduler + executor in their own process (ZMQ + msgpack boundary)
    enable_lora: bool = False
    max_loras: int = 8
    # TokenWeave
    tokenweave_mode: str = "overlap"
    tokenweave_config: Optional[str] = None
    tokenweave_threshold: Optional[int] = None
    tokenweave_transport: str = "auto"
    tokenweave_cuda_graphs: bool = False
    tokenweave_force_overlap: bool = False
    tokenweave_split_offset: Optional[int] = None
    tokenweave_attention_ctas: Optional[int] = None
    tokenweave_mlp_ctas: Optional[int] = None
    fuse_only_ctas: int = 16

    def create_engine_config(self) -> EngineConfig:
        model = resolve_model_config(self.model, None if self.dtype == "auto" else self.dtype,
                                     self.max_model_len, self.num_hidden_layers_override)
        if self.enable_expert_parallel and model.is_moe:
            if model.num_experts % self.tensor_parallel_size:
                raise ValueError("enable_expert_parallel needs num_experts divisible by tensor_parallel_size")
            model.expert_parallel = True
        max_len = model.max_model_len
        budget = self.max_num_batched_tokens or (8192 if self.enable_chunked_prefill else max(max_len, 8192))
        if self.quantization is None and model.checkpoint_quantization is not None:
            self.quantization = model.checkpoint_quantization        # an fp8 checkpoint runs on the fp8 GEMMs
        if self.quantization not in (None, "fp8", "int8"):
            raise ValueError(f"unknown quantization {self.quantization!r} (supported: fp8, int8)")
        if self.quantization and self.tokenweave_mode == "fused_gemm":
            raise ValueError("the fused GEMM+collective kernels take bf16 weights: use tokenweave_mode "
                             "overlap or fuse_only with quantization")
        load_format = self.load_format
        if load_format == "auto":
            load_format = "safetensors" if model.path else "dummy"
        return EngineConfig(
            model=model,
            cache=CacheConfig(self.block_size, self.gpu_memory_utilization, self.num_gpu_blocks_override,
                              self.enable_prefix_caching or self.kv_transfer_config is not None),   # the connector keys blocks by prefix hash
            parallel=ParallelConfig(self.tensor_parallel_size, self.distributed_executor_backend,
                                    self.disable_custom_all_reduce, data_parallel_size=self.data_parallel_size,
                                    data_parallel_rank=self.data_parallel_rank,
                                    pipeline_parallel_size=self.pipeline_parallel_size),
            scheduler=SchedulerConfig(budget, self.max_num_seqs, self.enable_chunked_prefill, max_len,
                                      self.scheduling_policy, max(0, int(self.long_prefill_token_threshold))),
            tokenweave=TokenWeaveConfig(mode=self.tokenweave_mode, config_path=self.tokenweave_config,
                                        overlap_threshold=self.tokenweave_threshold,
                                        transport=self.tokenweave_transport,
                                        use_cuda_graphs=self.tokenweave_cuda_graphs,
                                        fuse_only_ctas=self.fuse_only_ctas,
                                        force_overlap=self.tokenweave_force_overlap,
                                        split_offset=self.tokenweave_split_offset,
                                        attention_ctas=self.tokenweave_attention_ctas,
                                        mlp_ctas=self.tokenweave_mlp_ctas),
            load_format=load_format, quantization=self.quantization, seed=self.seed, device=self.device, enforce_eager=self.enforce_eager,
            tokenizer=self.tokenizer, skip_tokenizer_init=self.skip_tokenizer_init,
            disable_log_stats=self.disable_log_stats, enable_sleep_mode=self.enable_sleep_mode,
            speculative=self._speculative(), enable_lora=self._lora_checked(model), max_loras=self.max_loras,
            kv_transfer=self._kv_transfer(), engine_core_process=self.engine_core_process)

    def _kv_transfer(self):
        from .engine.kv_connector import KVTransferConfig
        return KVTransferConfig.from_user(self.kv_transfer_config)

    def _lora_checked(self, model) -> bool:
        if self.enable_lora and self.tokenweave_mode == "fused_gemm":
            raise ValueError("LoRA deltas are applied after the base GEMMs: use tokenweave_mode overlap or fuse_only")
        if self.enable_lora and self.quantization:
            raise ValueError("LoRA on quantised base weights is not supported")
        return self.enable_lora

    def _speculative(self):
        from .engine.spec_decode import SpecDecodeConfig
        value = self.speculative_config
        if isinstance(value, str):          # command line: a JSON object or a bare integer
            value = json.loads(value)
        return SpecDecodeConfig.from_user(value)

    @staticmethod
    def add_cli_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
        for f in dataclasses.fields(EngineArgs):
            flag = "--" + f.name.replace("_", "-")
            if f.type in ("bool", bool):
                parser.add_argument(flag, action=argparse.BooleanOptionalAction, default=f.default)
            else:
                typ = {"int": int, "float": float, "Optional[int]": int, "str": str, "Optional[str]": str}.get(
                    str(f.type), str)
                parser.add_argument(flag, type=typ, default=f.default)
        return parser

    @staticmethod
    def from_cli_args(ns: argparse.Namespace) -> "EngineArgs":
        names = {f.name for f in dataclasses.fields(EngineArgs)}
        return EngineArgs(**{k: v for k, v in vars(ns).items() if k in names})
