"""ctypes binding of ``tokenweave_b200/_C.so`` (see ``csrc/tw_kernels.h``).

The library is loaded on first use. On a machine with a GPU a missing library is an error, never a
silent fallback: the CUDA path of every op goes through this module.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path
from typing import Optional

_LIB_PATH = Path(__file__).resolve().parent.parent / "_C.so"
_lib: Optional[C.CDLL] = None
_lock = threading.Lock()

vp, ll, i32, f32, u64 = C.c_void_p, C.c_longlong, C.c_int, C.c_float, C.c_ulonglong

_SIGNATURES = {
    "tw_gemm_bf16": [vp, ll, vp, ll, ll, vp, ll, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, i32, vp, vp],
    "tw_gemm_bf16_grouped256": [vp, ll, vp, ll, ll, vp, ll, vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, vp, vp],
    "tw_rmsnorm": [vp, vp, vp, i32, i32, ll, ll, f32, i32, vp],
    "tw_rmsnorm_copy": [vp, vp, vp, i32, i32, ll, ll, f32, i32, vp],
    "tw_add_rmsnorm": [vp, vp, vp, i32, i32, ll, ll, f32, i32, vp],
    "tw_rope_kv_write": [vp, ll, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "tw_rope_kv_write_qknorm": [vp, ll, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, f32, vp],
    "tw_swiglu": [vp, ll, vp, ll, i32, i32, vp],
    "tw_embedding": [vp, vp, vp, ll, i32, i32, i32, i32, vp],
    "tw_argmax": [vp, ll, vp, i32, i32, vp],
    "tw_sample": [vp, ll, i32, i32, vp, vp, vp],
    "tw_gemm_fp8": [vp, ll, vp, ll, ll, vp, ll, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, i32, i32, i32, vp, vp],
    "tw_gemm_int8": [vp, ll, vp, ll, vp, ll, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp],
    "tw_quant_fp8": [vp, ll, vp, ll, vp, i32, i32, i32, i32, vp],
    "tw_rmsnorm_quant_fp8": [vp, vp, vp, vp, ll, vp, i32, i32, ll, ll, f32, i32, i32, vp],
    "tw_quant_int8": [vp, ll, vp, ll, vp, i32, i32, i32, i32, vp],
    "tw_rmsnorm_quant_int8": [vp, vp, vp, vp, ll, vp, i32, i32, ll, ll, f32, i32, i32, vp],
    "tw_gather_cache": [vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "tw_convert_fp8": [vp, vp, ll, f32, i32, vp],
    "tw_permute_cols": [vp, vp, vp, i32, i32, ll, ll, vp],
    "tw_activation": [vp, ll, vp, ll, i32, i32, i32, f32, vp],
    "tw_copy_pages": [vp, ll, vp, i32, vp],
    "tw_swap_pages": [vp, vp, ll, vp, i32, vp],
    "tw_merge_attn_states": [vp, vp, vp, vp, vp, vp, i32, i32, i32, vp],
    "tw_attn_prefill": [vp, ll, i32, vp, vp, i32, i32, vp, ll, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32,
                        f32, i32, i32, f32, vp, vp],
    "tw_attn_decode": [vp, ll, vp, vp, i32, vp, ll, vp, vp, vp, i32, vp, i32, i32, i32, i32, f32, i32, vp, vp,
                       i32, f32, vp],
    "tw_attn_decode_tc": [vp, ll, vp, vp, i32, i32, vp, ll, vp, vp, vp, i32, vp, i32, i32, i32, i32, f32, i32, vp, vp,
                          vp, vp],
    "tw_attn_decode_tc_persistent": [vp, ll, vp, vp, i32, i32, vp, ll, vp, vp, vp, i32, vp, i32, i32, i32, i32, f32,
                                     i32, vp, vp, i32, vp, vp],
    "tw_moe_router": [vp, ll, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp],
    "tw_moe_align": [vp, i32, i32, i32, vp, vp, vp, i32, vp, vp],
    "tw_moe_scatter": [vp, ll, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp],
    "tw_moe_combine": [vp, vp, vp, ll, i32, i32, i32, vp],
    "tw_fused_rs_norm_ag": [vp, vp, vp, i32, i32, i32, u64, vp, ll, vp, ll, vp, i32, i32, f32, i32, i32, i32,
                            vp],
    "tw_collective": [vp, vp, vp, i32, i32, i32, u64, vp, ll, ll, i32, i32, vp],
    "tw_oneshot_allreduce": [vp, vp, i32, i32, i32, u64, vp, ll, ll, vp, i32, vp],
    "tw_wait_probe": [vp, u64, vp, vp],
    "tw_gemm_rs_norm": [vp, ll, vp, ll, i32, i32, i32, vp, vp, vp, vp, vp, i32, i32, u64, vp, ll, i32, vp, ll, vp, f32,
                        i32, i32, vp],
    "tw_ag_gemm": [vp, vp, ll, ll, vp, ll, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, i32, i32, u64, vp, ll, i32, i32,
                   i32, vp],
}


class NativeLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists():
            raise NativeLibraryError(
                f"{_LIB_PATH} is missing: build it with `python -m tokenweave_b200.build` "
                "(the CUDA ops have no fallback on a GPU)")
        lib = C.CDLL(str(_LIB_PATH))
        lib.tw_last_error.restype = C.c_char_p
        lib.tw_last_error.argtypes = []
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = argtypes
        for name in dir(OptionalSymbols):
            if name.startswith("tw_"):
                try:
                    fn = getattr(lib, name)
                except AttributeError:
                    continue
                fn.restype = C.c_int
                fn.argtypes = getattr(OptionalSymbols, name)
        _lib = lib
    return _lib


class OptionalSymbols:
    """Entry points that newer builds of the library export; bound when present."""


_launches = 0
_timing = None      # name -> list of (start event, end event) while op timing is on


def launch_count() -> int:
    """Number of launcher calls made so far by this process (each is at least one kernel launch)."""
    return _launches


def enable_op_timing(on: bool = True) -> None:
    """Bracket every launcher call with CUDA events (the layer-wise profile of ``utils/profiler.py``)."""
    global _timing
    _timing = {} if on else None


def op_timing_summary(reset: bool = True) -> dict:
    """{op name: (calls, total milliseconds)} of the launches recorded since timing was enabled."""
    import torch
    global _timing
    if _timing is None:
        return {}
    torch.cuda.synchronize()
    out = {k: (len(v), sum(a.elapsed_time(b) for a, b in v)) for k, v in _timing.items()}
    if reset:
        _timing = {}
    return out


def call(name: str, *args, tag: str = "") -> None:
    global _launches
    lib = load()
    _launches += 1
    if _timing is not None:
        import torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rc = getattr(lib, name)(*args)
        b.record()
        _timing.setdefault(name + tag, []).append((a, b))
    else:
        rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.tw_last_error()
        raise NativeLibraryError(f"{name} failed: {msg.decode() if msg else 'unknown error'}")
