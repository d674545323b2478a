"""Weight loading: HuggingFace safetensors checkpoints (sharded, with or without an index file),
``.bin``/``.pt`` state dicts, and random initialisation for performance runs.

Counterpart of vllm/model_executor/model_loader/loader.py:330-500. Tensors are streamed file by file
and narrowed to this rank's shard by each parameter's ``weight_loader`` before they reach the GPU, so
peak host memory is one checkpoint shard.
"""
from __future__ import annotations

import glob
import json
import os
from typing import Iterator, Optional

import torch

from ..config import EngineConfig
from ..utils.logging import init_logger

logger = init_logger(__name__)


def iter_checkpoint(path: str) -> Iterator[tuple[str, torch.Tensor]]:
    st_files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    index = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            wanted = set(json.load(f)["weight_map"].values())
        st_files = [f for f in st_files if os.path.basename(f) in wanted]
    if st_files:
        from safetensors import safe_open
        for fname in st_files:
            with safe_open(fname, framework="pt", device="cpu") as f:
                for key in f.keys():
                    yield key, f.get_tensor(key)
        return
    pt_files = sorted(glob.glob(os.path.join(path, "*.bin")) + glob.glob(os.path.join(path, "*.pt")))
    if not pt_files:
        raise FileNotFoundError(f"no *.safetensors, *.bin or *.pt weights under {path}")
    for fname in pt_files:
        state = torch.load(fname, map_location="cpu", weights_only=True)
        yield from state.items()
        del state


_FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)
_SCALE_SUFFIXES = (".weight_scale", ".weight_scale_inv")
_DROPPED_SUFFIXES = (".input_scale", ".k_scale", ".v_scale", ".q_scale", ".kv_scale")


def dequantize_fp8(weight: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp8 weight x its scale in fp32: per tensor (one value), per output channel (``[N]`` / ``[N, 1]``) or per
    block (``[ceil(N / b), ceil(K / b)]``, the 128 x 128 block layout of block-quantised checkpoints)."""
    w, s = weight.float(), scale.float()
    if s.numel() == 1:
        return w * s.reshape(())
    if s.ndim == 1 or (s.ndim == 2 and s.shape[1] == 1):
        return w * s.reshape(-1, 1)
    if s.ndim == 2:
        br, bc = -(-w.shape[0] // s.shape[0]), -(-w.shape[1] // s.shape[1])
        full = s.repeat_interleave(br, 0)[: w.shape[0]].repeat_interleave(bc, 1)[:, : w.shape[1]]
        return w * full
    raise ValueError(f"fp8 scale of shape {tuple(s.shape)} for a weight of shape {tuple(w.shape)}")


_AWQ_NIBBLE_TO_COLUMN = (0, 2, 4, 6, 1, 3, 5, 7)     # nibble i of a packed word holds output column 8 c + this


def _unpack_columns(packed: torch.Tensor, bits: int, order=None) -> torch.Tensor:
    """int32 ``[R, C]`` whose words pack ``32 / bits`` values along the columns -> int32 ``[R, C * 32 / bits]``;
    ``order[i]`` is the column (within its group) that field i of a word holds (default: i)."""
    per = 32 // bits
    shifts = torch.arange(per, dtype=torch.int32) * bits
    vals = (packed.to(torch.int32).unsqueeze(-1) >> shifts) & ((1 << bits) - 1)       # [R, C, per] by field
    if order is not None:
        out = torch.empty_like(vals)
        out[..., list(order)] = vals
        vals = out
    return vals.reshape(packed.shape[0], -1)


def dequantize_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, group_size: int) -> torch.Tensor:
    """AWQ GEMM layout (4 bits): ``qweight`` int32 ``[K, N / 8]`` and ``qzeros`` int32 ``[K / g, N / 8]`` pack eight
    output columns per word in the order 0, 2, 4, 6, 1, 3, 5, 7; ``scales`` ``[K / g, N]``. Returns the ``[N, K]``
    fp32 weight ``(q - z) * s`` (the arithmetic of the reference's ``awq_dequantize``,
    csrc/quantization/awq/gemm_kernels.cu)."""
    q = _unpack_columns(qweight, 4, _AWQ_NIBBLE_TO_COLUMN)
    z = _unpack_columns(qzeros, 4, _AWQ_NIBBLE_TO_COLUMN)
    g = group_size if group_size > 0 else q.shape[0]
    z = z.repeat_interleave(g, 0)[: q.shape[0]]
    s = scales.float().repeat_interleave(g, 0)[: q.shape[0]]
    return ((q - z).float() * s).t().contiguous()


def dequantize_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, g_idx: Optional[torch.Tensor],
                    bits: int, group_size: int, zeros_plus_one: bool) -> torch.Tensor:
    """GPTQ layout: ``qweight`` int32 ``[K * bits / 32, N]`` packs consecutive INPUT rows per word, ``qzeros`` int32
    ``[K / g, N * bits / 32]`` packs consecutive output columns, ``scales`` ``[K / g, N]``, ``g_idx`` ``[K]`` names the
    group of every input row (activation order; absent: row // group size). Returns the ``[N, K]`` fp32 weight
    ``(q - z) * s`` (the reference's csrc/quantization/gptq/q_gemm.cu reconstruction)."""
    q = _unpack_columns(qweight.t().contiguous(), bits).t()                  # [K, N]
    z = _unpack_columns(qzeros, bits)                                         # [K / g, N]
    if zeros_plus_one:
        z = z + 1          # no wrap-around: a stored 15 means 16, as in the reference's kernel
    K = q.shape[0]
    if g_idx is None:
        g = group_size if group_size > 0 else K
        idx = torch.arange(K) // g
    else:
        idx = g_idx.long()
    return ((q - z[idx]).float() * scales.float()[idx]).t().contiguous()


_PACKED_SUFFIXES = (".qweight", ".qzeros", ".scales", ".g_idx")


def unpacked_stream(weights: Iterator[tuple[str, torch.Tensor]], packing: Optional[dict]):
    """Expands the packed tensors of an AWQ / GPTQ checkpoint (``<linear>.qweight / qzeros / scales [/ g_idx]``) into
    ``<linear>.weight`` in fp32 as soon as a linear's tensors are complete; everything else passes through. The
    engine then runs the model in its 16-bit dtype (or re-quantises to fp8 / int8 if asked to): weight-only 4-bit
    GEMMs are not built."""
    if not packing:
        yield from weights
        return
    need = {"qweight", "qzeros", "scales"} | ({"g_idx"} if packing["method"] == "gptq" else set())
    parts: dict[str, dict[str, torch.Tensor]] = {}

    def expand(d):
        if packing["method"] == "awq":
            return dequantize_awq(d["qweight"], d["qzeros"], d["scales"], packing["group_size"])
        return dequantize_gptq(d["qweight"], d["qzeros"], d["scales"], d.get("g_idx"), packing["bits"],
                               packing["group_size"], packing["zeros_plus_one"])

    for name, t in weights:
        if not name.endswith(_PACKED_SUFFIXES):
            yield name, t
            continue
        stem, kind = name.rsplit(".", 1)
        d = parts.setdefault(stem, {})
        d[kind] = t
        if need <= set(d):
            yield stem + ".weight", expand(parts.pop(stem))
    for stem, d in parts.items():            # GPTQ files without g_idx tensors end up here
        missing = {"qweight", "qzeros", "scales"} - set(d)
        if missing:
            raise ValueError(f"{stem}: packed checkpoint lacks {sorted(missing)}")
        yield stem + ".weight", expand(d)


def dequantized_stream(weights: Iterator[tuple[str, torch.Tensor]]) -> Iterator[tuple[str, torch.Tensor]]:
    """Pass-through for ordinary checkpoints. For fp8 checkpoints (``weight`` stored as e4m3 next to a
    ``weight_scale`` / ``weight_scale_inv``; the FP8 and compressed-tensors layouts the reference reads in
    vllm/model_executor/layers/quantization/fp8.py) every weight comes out as fp32 = fp8 x scale (the parameter copy rounds it to the model's dtype), whichever of
    the two tensors the file lists first; static activation and KV scales are dropped (activations are quantised
    dynamically here). With ``quantization="fp8"`` the layers are then re-quantised per output channel, which
    reproduces a per-channel checkpoint exactly."""
    pending_w: dict[str, torch.Tensor] = {}
    pending_s: dict[str, torch.Tensor] = {}
    for name, t in weights:
        if name.endswith(_DROPPED_SUFFIXES):
            continue
        stem = None
        if name.endswith(_SCALE_SUFFIXES):
            stem = name.rsplit(".", 1)[0]
            pending_s[stem] = t
        elif name.endswith(".weight") and t.dtype in _FP8_DTYPES:
            stem = name[: -len(".weight")]
            pending_w[stem] = t
        else:
            yield name, t
            continue
        if stem in pending_w and stem in pending_s:
            yield stem + ".weight", dequantize_fp8(pending_w.pop(stem), pending_s.pop(stem))
    for stem, w in pending_w.items():          # an fp8 tensor without a scale: its values are the weights
        yield stem + ".weight", w.float()


def load_model_weights(model, config: EngineConfig) -> None:
    fmt = config.load_format
    if fmt == "dummy" or (fmt == "auto" and not config.model.path):
        model.init_dummy_weights(config.seed)
    elif fmt == "sharded_state":
        # every rank reads back exactly the parameters it wrote with ``LLM.save_sharded_state``: no resharding,
        # no name mapping (vllm/model_executor/model_loader/loader.py ``ShardedStateLoader``)
        from safetensors.torch import load_file
        from ..parallel.state import get_tp
        fname = os.path.join(config.model.path or "", f"rank_{get_tp().global_rank}.safetensors")
        if not os.path.exists(fname):
            raise FileNotFoundError(f"load_format='sharded_state' needs {fname} (written by LLM.save_sharded_state)")
        state = load_file(fname)
        params = dict(model.named_parameters())
        missing = sorted(set(params) - set(state))
        if missing:
            raise ValueError(f"{fname} lacks {len(missing)} parameters of this rank (first: {missing[0]}); it was "
                             f"saved under another parallel layout")
        for n, p_ in params.items():
            if tuple(state[n].shape) != tuple(p_.shape):
                raise ValueError(f"{fname}: {n} has shape {tuple(state[n].shape)}, this rank expects {tuple(p_.shape)}")
            p_.data.copy_(state[n])
        logger.info("loaded %d sharded tensors from %s", len(params), fname)
    else:
        if not config.model.path:
            raise ValueError(f"load_format={fmt!r} needs a checkpoint directory")
        loaded = model.load_weights(dequantized_stream(unpacked_stream(iter_checkpoint(config.model.path),
                                                                       config.model.checkpoint_packing)))
        logger.info("loaded %d tensors from %s", len(loaded), config.model.path)
    if config.quantization in ("fp8", "int8"):
        quantize_linears_fp8_(model, config.quantization)


def quantize_linears_fp8_(model, kind: str = "fp8") -> int:
    """Online fp8 quantisation of a loaded bf16 model: every tensor-parallel linear of the decoder
    layers gets an e4m3 weight with per-output-channel scales (the reference quantises bf16
    checkpoints the same way when ``quantization="fp8"`` meets an unquantised checkpoint,
    vllm/model_executor/layers/quantization/fp8.py). The LM head, the embedding, the MoE router and
    the expert weights stay bf16. ``kind="int8"``: symmetric int8 instead of e4m3. Returns the number of layers
    converted."""
    from ..layers.linear import _QuantizableLinear
    from ..layers.embedding import ParallelLMHead
    n = 0
    for name, mod in model.named_modules():
        if isinstance(mod, _QuantizableLinear) and not isinstance(mod, ParallelLMHead) and "gate." not in name + ".":
            mod.quantize_int8_() if kind == "int8" else mod.quantize_fp8_()
            n += 1
    logger.info("quantised %d linear layers to %s (per-channel weight scales)", n, kind)
    return n


def save_hf_checkpoint(state: dict[str, torch.Tensor], hf_config: dict, path: str, shards: int = 1) -> None:
    """Write tensors in HuggingFace layout (used by tests and by the sharded-state export)."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf_config, f)
    names = sorted(state)
    per = (len(names) + shards - 1) // shards
    weight_map = {}
    for s in range(shards):
        part = {n: state[n].contiguous() for n in names[s * per:(s + 1) * per]}
        fname = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        save_file(part, os.path.join(path, fname))
        weight_map.update({n: fname for n in part})
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
