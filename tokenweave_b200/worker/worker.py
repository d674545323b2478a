"""Worker: one per GPU. Binds the device, joins the process group, loads the model, sizes and allocates
the KV cache, and executes steps.

Counterpart of vllm/v1/worker/gpu_worker.py:91-252.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import envs, ops
from ..config import EngineConfig
from ..parallel import state as pstate
from ..utils.logging import init_logger
from .model_runner import ModelRunner, StepData, StepResult

logger = init_logger(__name__)


class Worker:
    def __init__(self, config: EngineConfig, rank: int = 0, local_rank: Optional[int] = None,
                 init_method: Optional[str] = None):
        self.config = config
        self.rank = rank
        self.local_rank = rank if local_rank is None else local_rank
        self.init_method = init_method
        self.runner: Optional[ModelRunner] = None
        self.profiler = None

    def init_device(self) -> None:
        world = self.config.parallel.world_size
        dev_kind = self.config.resolved_device()
        if world > 1:
            tp = pstate.init_distributed(self.rank, world, self.local_rank, dev_kind, self.init_method,
                                         tp_size=self.config.parallel.tensor_parallel_size)
        else:
            if dev_kind == "cuda":
                torch.cuda.set_device(self.local_rank)
                dev = torch.device("cuda", self.local_rank)
            else:
                dev = torch.device("cpu")
            tp = pstate.set_single_process(dev)
        self.device = tp.device
        torch.manual_seed(self.config.seed)
        self.runner = ModelRunner(self.config, self.device)

    def _sleep_pool(self, tag: int):
        """Allocation context of sleep mode: the VMM pool of ``tag`` on a GPU with ``enable_sleep_mode``,
        else nothing."""
        import contextlib
        if self.config.enable_sleep_mode and self.device.type == "cuda":
            from ..utils.sleep_allocator import SleepAllocator
            return SleepAllocator.get().use_pool(tag)
        return contextlib.nullcontext()

    def load_model(self) -> None:
        from ..utils.sleep_allocator import TAG_WEIGHTS
        self.runner.load_model(embedding_parallel=bool(int(os.getenv("TW_EMBEDDING_PARALLEL", "0"))),
                               weights_pool=self._sleep_pool(TAG_WEIGHTS))

    def determine_num_blocks(self) -> int:
        """KV blocks that fit in what is left of ``gpu_memory_utilization`` after weights and workspaces."""
        cache = self.config.cache
        if cache.num_gpu_blocks is not None:
            return cache.num_gpu_blocks
        per_block = self.runner.model.kv_cache_bytes_per_block(cache.block_size)
        if self.device.type != "cuda":
            want = self.config.scheduler.max_num_batched_tokens * 4 // cache.block_size + 16
            return max(16, want)
        torch.cuda.synchronize()
        free, total = torch.cuda.mem_get_info(self.device)
        used_by_others = total - free - torch.cuda.memory_reserved(self.device)
        budget = total * cache.gpu_memory_utilization - torch.cuda.memory_reserved(self.device) - max(0, used_by_others)
        budget -= 2 << 30     # logits, sampler temporaries, NCCL buffers
        n = int(budget // per_block)
        if n < 4:
            raise RuntimeError(f"not enough GPU memory for the KV cache ({budget / 1e9:.1f} GB left, "
                               f"{per_block / 1e6:.1f} MB per block)")
        max_useful = (self.config.scheduler.max_model_len * self.config.scheduler.max_num_seqs) // cache.block_size + 64
        return min(n, max_useful)

    def init_kv_cache(self, num_blocks: int) -> None:
        from ..utils.sleep_allocator import TAG_KV_CACHE
        with self._sleep_pool(TAG_KV_CACHE):
            self.runner.init_kv_cache(num_blocks)
        logger.info("KV cache: %d blocks of %d tokens", num_blocks, self.config.cache.block_size)

    def execute_model(self, step: StepData) -> StepResult:
        return self.runner.execute_model(step)

    def check_health(self) -> bool:
        if self.device.type == "cuda":
            ops.check_status(self.device)
        return True

    def reset_comm_state(self) -> None:
        """Collective: put signal pads, tile flags, epochs and the status word back to their start state after a
        step ended with a non-zero status word (``EngineCore`` is dead by then; a supervisor that wants to go on
        calls this on all workers and builds a new core on the same executor)."""
        rt = self.runner.model.rt if self.runner is not None and self.runner.model is not None else None
        if rt is not None:
            rt.comm.reset_after_failure()

    # ---- profiling hooks (LLM.start_profile / stop_profile) ----
    def profile(self, start: bool) -> None:
        trace_dir = envs.TW_TORCH_PROFILER_DIR
        if trace_dir is None:
            raise RuntimeError("set TW_TORCH_PROFILER_DIR to enable the torch profiler")
        if start:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if self.device.type == "cuda":
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self.profiler = torch.profiler.profile(
                activities=acts, with_stack=True,
                on_trace_ready=torch.profiler.tensorboard_trace_handler(trace_dir, use_gzip=True))
            self.profiler.start()
        elif self.profiler is not None:
            self.profiler.stop()
            self.profiler = None

    # ---- sleep / wake (weights to host memory, KV cache dropped) ----
    def sleep(self, level: int = 1) -> None:
        if self.config.enable_sleep_mode and self.device.type == "cuda":
            # VMM path: physical memory of weights and KV cache is released, addresses stay valid.
            # Level 1 keeps the weights in pinned host memory; level 2 discards them too.
            from ..utils.sleep_allocator import TAG_WEIGHTS, SleepAllocator
            alloc = SleepAllocator.get()
            before = torch.cuda.mem_get_info(self.device)[0]
            alloc.sleep(offload_tags=(TAG_WEIGHTS,) if level == 1 else ())
            self._vmm_sleep_level = level
            logger.info("sleep level %d freed %.2f GB of device memory (%.2f GB held on the host)", level,
                        (torch.cuda.mem_get_info(self.device)[0] - before) / 1e9, alloc.host_bytes() / 1e9)
            return
        model = self.runner.model
        self._sleeping = {}
        self._param_shapes = {n: tuple(p.shape) for n, p in model.named_parameters()}
        for name, p in model.named_parameters():
            if level == 1:
                host = torch.empty(p.shape, dtype=p.dtype, pin_memory=(self.device.type == "cuda"))
                host.copy_(p.data)
                self._sleeping[name] = host
            p.data = torch.empty(0, dtype=p.dtype, device=self.device)
        self._kv_shape = None
        for layer in model.layers:
            if layer.attn.k_cache is not None:
                self._kv_shape = tuple(layer.attn.k_cache.shape)
            layer.attn.bind_kv_cache(None, None)
        if self.device.type == "cuda":
            torch.cuda.synchronize()
            torch.cuda.empty_cache()

    def wake_up(self) -> None:
        model = self.runner.model
        level = getattr(self, "_vmm_sleep_level", None)
        if level is not None:
            from ..utils.sleep_allocator import SleepAllocator
            SleepAllocator.get().wake_up()
            if level >= 2:        # the weights were discarded: reload (or re-draw) them into the same tensors
                from ..models.loader import load_model_weights
                if self.config.quantization:
                    raise RuntimeError("sleep level 2 with online quantisation needs a fresh engine")
                load_model_weights(model, self.config)
            for layer in model.layers:      # the KV cache came back uninitialised
                if layer.attn.k_cache is not None:
                    layer.attn.k_cache.zero_()
                    layer.attn.v_cache.zero_()
            torch.cuda.synchronize()
            self._vmm_sleep_level = None
            return
        saved = getattr(self, "_sleeping", None)
        if saved is None:
            return
        if saved:
            for name, p in model.named_parameters():
                p.data = saved[name].to(self.device, non_blocking=True)
        else:
            # level 2 discarded the weights: bring them back from the checkpoint (or re-draw them)
            from ..models.loader import load_model_weights
            for name, p in model.named_parameters():
                p.data = torch.empty(self._param_shapes[name], dtype=p.dtype, device=self.device)
            load_model_weights(model, self.config)
        if self._kv_shape is not None:
            self.runner.init_kv_cache(self._kv_shape[0])
        self._sleeping = None
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    # ---- KV connector (engine/kv_connector.py): blocks to / from the external store -------------------------
    def _kv_connector(self):
        if getattr(self, "_connector", None) is None:
            from ..engine.kv_connector import kv_fingerprint, make_connector
            tp = pstate.get_tp()
            self._connector = make_connector(self.config.kv_transfer, tp.global_rank, tp.global_size,
                                             kv_fingerprint(self.config))
        return self._connector

    def save_kv_blocks(self, items: list) -> None:
        """items: (block id, block hash); this rank's slice of every local layer goes into one file per block."""
        conn = self._kv_connector()
        layers = self.runner.model.layers
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)       # the step that filled the blocks has completed
        for block, h in items:
            if conn.available(h):
                continue
            k = torch.stack([layer.attn.k_cache[block] for layer in layers])
            v = torch.stack([layer.attn.v_cache[block] for layer in layers])
            conn.save_block(h, k, v)

    def load_kv_blocks(self, items: list) -> None:
        conn = self._kv_connector()
        layers = self.runner.model.layers
        want = (len(layers),) + tuple(layers[0].attn.k_cache.shape[1:])
        for block, h in items:
            k, v = conn.load_block(h, want)
            for i, layer in enumerate(layers):
                layer.attn.k_cache[block].copy_(k[i], non_blocking=True)
                layer.attn.v_cache[block].copy_(v[i], non_blocking=True)

    def set_capture_hidden(self, on: bool) -> None:
        """Pooling support: keep the final-norm hidden state at every request's first sampled position."""
        self.runner.capture_hidden = bool(on)
        self.runner.captured_hidden = {}

    def take_captured_hidden(self) -> dict:
        out, self.runner.captured_hidden = self.runner.captured_hidden, {}
        return out

    def save_sharded_state(self, path: str) -> None:
        from safetensors.torch import save_file
        os.makedirs(path, exist_ok=True)
        state = {n: p.detach().cpu().contiguous() for n, p in self.runner.model.named_parameters()}
        save_file(state, os.path.join(path, f"rank_{self.rank}.safetensors"))
        src = self.config.model.path
        if self.rank == 0 and src and os.path.isdir(src) and os.path.abspath(src) != os.path.abspath(path):
            import shutil      # the directory then loads on its own with load_format="sharded_state"
            for name in os.listdir(src):
                if name.endswith(".json") or name.startswith("tokenizer") or name.endswith(".model"):
                    if "safetensors.index" not in name:
                        shutil.copy(os.path.join(src, name), os.path.join(path, name))

    def load_sharded_state(self, path: str) -> None:
        from safetensors.torch import load_file
        state = load_file(os.path.join(path, f"rank_{self.rank}.safetensors"))
        for n, p in self.runner.model.named_parameters():
            p.data.copy_(state[n])

    def shutdown(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        if self.runner is not None:
            # captured graphs hold NCCL kernels (the logits gather) and pool memory: release them before the
            # communicator goes away, or its destruction waits on them
            self.runner.release_graphs()
        if self.runner is not None and self.runner.model is not None and self.runner.model.rt is not None:
            try:
                if self.runner.model.rt.comm.pynccl is not None:
                    self.runner.model.rt.comm.pynccl.destroy()
                    self.runner.model.rt.comm.pynccl = None
                self.runner.model.rt.staging.close()
            except Exception as e:       # tear-down must not mask the caller's error
                logger.warning("symmetric buffer tear-down failed: %s", e)
        self.runner = None
        pstate.destroy_distributed()
