"""AWQ and GPTQ checkpoints: the packed tensors are expanded while loading and the engine generates what the
naive model does on the expanded weights. The packers below write the layouts from their definitions (AWQ: eight
output columns per word in the order 0, 2, 4, 6, 1, 3, 5, 7; GPTQ: eight input rows per word, zero points stored
minus one, an optional permutation of the input rows over the groups)."""
import pytest
import torch

from tokenweave_b200 import LLM, SamplingParams
from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
from tokenweave_b200.models.loader import dequantize_awq, dequantize_gptq, save_hf_checkpoint

from tw_testing import hf_config_dict, make_hf_state, naive_logits

GROUP = 32


def _quantise(w, bits, g_idx):
    """[N, K] fp32 -> integer codes [K, N], zero points [K / g, N], scales [K / g, N] (asymmetric, per group)."""
    K = w.shape[1]
    n_groups = K // GROUP
    wt = w.t().contiguous()                                   # [K, N]
    q = torch.empty_like(wt, dtype=torch.int32)
    zeros = torch.empty(n_groups, w.shape[0], dtype=torch.int32)
    scales = torch.empty(n_groups, w.shape[0])
    top = (1 << bits) - 1
    for g in range(n_groups):
        rows = (g_idx == g).nonzero().flatten()
        blk = wt[rows]
        lo, hi = blk.amin(0), blk.amax(0)
        s = ((hi - lo) / top).clamp_min(1e-8)
        z = torch.round(-lo / s).clamp(1, top).to(torch.int32)         # zero point 0 has no GPTQ-v1 encoding
        q[rows] = torch.round(blk / s + z).clamp(0, top).to(torch.int32)
        zeros[g], scales[g] = z, s
    return q, zeros, scales


def _to_i32(word64):
    return torch.where(word64 >= 2 ** 31, word64 - 2 ** 32, word64).to(torch.int32)


def _pack(vals, bits, order=None):
    per = 32 // bits
    v = vals.reshape(vals.shape[0], -1, per).to(torch.int64)
    if order is not None:
        v = v[..., list(order)]
    word = torch.zeros(v.shape[:2], dtype=torch.int64)
    for i in range(per):
        word |= v[..., i] << (bits * i)
    return _to_i32(word)


def _awq_tensors(w):
    g_idx = torch.arange(w.shape[1]) // GROUP
    q, z, s = _quantise(w, 4, g_idx)
    order = (0, 2, 4, 6, 1, 3, 5, 7)
    return {"qweight": _pack(q, 4, order), "qzeros": _pack(z, 4, order), "scales": s.half()}, (q, z, s, g_idx)


def _gptq_tensors(w, bits, act_order, seed):
    K = w.shape[1]
    g_idx = torch.arange(K) // GROUP
    if act_order:
        g_idx = g_idx[torch.randperm(K, generator=torch.Generator().manual_seed(seed))]
    q, z, s = _quantise(w, bits, g_idx)
    t = {"qweight": _pack(q.t().contiguous(), bits).t().contiguous(), "qzeros": _pack(z - 1, bits), "scales": s.half(),
         "g_idx": g_idx.to(torch.int32)}
    return t, (q, z, s, g_idx)


def _expected(q, z, s, g_idx):
    return ((q - z[g_idx]).float() * s.half().float()[g_idx]).t()


@pytest.mark.parametrize("bits,act_order", [(4, False), (4, True), (8, True)])
def test_gptq_unpacking(bits, act_order):
    w = torch.randn(48, 128, generator=torch.Generator().manual_seed(0))
    t, parts = _gptq_tensors(w, bits, act_order, 1)
    got = dequantize_gptq(t["qweight"], t["qzeros"], t["scales"], t["g_idx"], bits, GROUP, True)
    torch.testing.assert_close(got, _expected(*parts), rtol=0, atol=0)
    assert (got - w).abs().max() < (0.35 if bits == 4 else 0.03)
    if not act_order:        # without g_idx the groups are consecutive rows
        got2 = dequantize_gptq(t["qweight"], t["qzeros"], t["scales"], None, bits, GROUP, True)
        torch.testing.assert_close(got2, got, rtol=0, atol=0)


def test_awq_unpacking():
    w = torch.randn(48, 128, generator=torch.Generator().manual_seed(2))
    t, parts = _awq_tensors(w)
    got = dequantize_awq(t["qweight"], t["qzeros"], t["scales"], GROUP)
    torch.testing.assert_close(got, _expected(*parts), rtol=0, atol=0)
    assert (got - w).abs().max() < 0.35


@pytest.mark.parametrize("method", ["awq", "gptq"])
def test_engine_serves_packed_checkpoints(tmp_path, method):
    cfg = ModelConfig(name="tiny-llama", **dict(MODEL_PRESETS["tiny-llama"], intermediate_size=704))   # 22 groups
    st = make_hf_state(cfg, seed=13)
    packed, expanded = {}, {}
    for name, w in st.items():
        if name.endswith("_proj.weight"):
            stem = name[: -len(".weight")]
            t, parts = _awq_tensors(w.float()) if method == "awq" else _gptq_tensors(w.float(), 4, True, len(packed))
            packed.update({f"{stem}.{k}": v for k, v in t.items()})
            expanded[name] = _expected(*parts)
        else:
            packed[name] = w
            expanded[name] = w
    hf = hf_config_dict(cfg)
    hf["quantization_config"] = ({"quant_method": "awq", "bits": 4, "group_size": GROUP, "version": "GEMM", "zero_point": True}
                                 if method == "awq" else
                                 {"quant_method": "gptq", "bits": 4, "group_size": GROUP, "desc_act": True, "sym": False})
    ckpt = str(tmp_path / "ckpt")
    save_hf_checkpoint(packed, hf, ckpt)
    llm = LLM(ckpt, dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=64)
    assert llm.llm_engine.config.model.checkpoint_packing["method"] == method
    prompt = list(range(5, 45))
    out = llm.generate([prompt], SamplingParams(temperature=0, max_tokens=4, ignore_eos=True))[0]
    seq = list(prompt)
    for _ in range(4):
        seq.append(int(naive_logits(cfg, expanded, seq)[-1].argmax()))
    assert out.outputs[0].token_ids == seq[len(prompt):]
    llm.shutdown()
