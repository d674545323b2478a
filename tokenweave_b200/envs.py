"""Environment variables, read lazily (the counterpart of vllm/envs.py:143-781).

``envs.TW_X`` evaluates the variable at access time, so tests and launch scripts can change it.
"""
from __future__ import annotations

import os
from typing import Any, Callable

_VARS: dict[str, Callable[[], Any]] = {
    # log level of the "tokenweave_b200" logger
    "TW_LOGGING_LEVEL": lambda: os.getenv("TW_LOGGING_LEVEL", "INFO"),
    # overrides the split offset of the TokenWeave config file (reference: TOKENWEAVE_SPLIT_OFFSET)
    "TW_SPLIT_OFFSET": lambda: (int(os.environ["TW_SPLIT_OFFSET"]) if "TW_SPLIT_OFFSET" in os.environ
                                else (int(os.environ["TOKENWEAVE_SPLIT_OFFSET"])
                                      if "TOKENWEAVE_SPLIT_OFFSET" in os.environ else None)),
    # overrides of the communication SM budgets (used by the config generator sweeps)
    "TW_MAX_CTAS_ATTN": lambda: int(os.environ["TW_MAX_CTAS_ATTN"]) if "TW_MAX_CTAS_ATTN" in os.environ else None,
    "TW_MAX_CTAS_MLP": lambda: int(os.environ["TW_MAX_CTAS_MLP"]) if "TW_MAX_CTAS_MLP" in os.environ else None,
    # directory for torch profiler traces; enables LLM.start_profile/stop_profile
    "TW_TORCH_PROFILER_DIR": lambda: os.getenv("TW_TORCH_PROFILER_DIR"),
    # emit NVTX ranges around every split / stage of the overlap schedule
    "TW_NVTX": lambda: os.getenv("TW_NVTX", "0") == "1",
    # symmetric-memory provider: "native" (own VMM allocator) or "torch"
    "TW_SYMM_PROVIDER": lambda: os.getenv("TW_SYMM_PROVIDER", "torch"),
    # disable NVLS multimem even when available (peer loads/stores instead)
    "TW_DISABLE_NVLS": lambda: os.getenv("TW_DISABLE_NVLS", "0") == "1",
    # worker process start method for the multiprocess executor
    "TW_WORKER_MULTIPROC_METHOD": lambda: os.getenv("TW_WORKER_MULTIPROC_METHOD", "spawn"),
    # seconds before an execute_model RPC to the workers is declared failed
    "TW_EXECUTE_MODEL_TIMEOUT_S": lambda: float(os.getenv("TW_EXECUTE_MODEL_TIMEOUT_S", "30")),
    "TW_RPC_TIMEOUT_S": lambda: float(os.getenv("TW_RPC_TIMEOUT_S", "180")),
    # trace every Python function call of the package to this file (debugging aid)
    "TW_TRACE_FUNCTION": lambda: os.getenv("TW_TRACE_FUNCTION"),
    # decode attention kernel: "1" tensor cores where they apply (default), "0" the SIMT kernel everywhere,
    # "persistent" the tensor-core kernel with one CTA per SM walking the work items (read by ops at import)
    "TW_DECODE_TC": lambda: os.getenv("TW_DECODE_TC", "1"),
    # vocabulary-parallel instead of replicated embedding table
    "TW_EMBEDDING_PARALLEL": lambda: os.getenv("TW_EMBEDDING_PARALLEL", "0") == "1",
    # NCCL baseline collectives and the logits gather through the package's own communicator (parallel/pynccl.py)
    # instead of torch.distributed; "0" leaves the process group in charge
    "TW_USE_PYNCCL": lambda: os.getenv("TW_USE_PYNCCL", "1") == "1",
    # libnccl for the ctypes binding (parallel/pynccl.py); default: the one torch ships
    "TW_NCCL_SO_PATH": lambda: os.getenv("TW_NCCL_SO_PATH"),
    # CUDA graphs: sights of a step shape that mixes prefill chunks with decode rows (or prefills several sequences)
    # before it is captured; decode-only steps and single-sequence prefills are captured on their second sight
    "TW_GRAPH_MIXED_SIGHTS": lambda: int(os.getenv("TW_GRAPH_MIXED_SIGHTS", "4")),
    # where the artifact scripts write their CSV / JSON results
    "TW_RESULTS_DIR": lambda: os.getenv("TW_RESULTS_DIR", "results"),
    # port range start for rendezvous when none is given
    "TW_PORT": lambda: int(os.getenv("TW_PORT", "29611")),
}


def __getattr__(name: str) -> Any:
    if name in _VARS:
        return _VARS[name]()
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return list(_VARS)
