"""End-to-end model correctness on CPU in fp32: the engine (paged cache, chunked prefill, token-split
schedule, HF checkpoint loading) against a naive dense forward of the same weights."""
import os

import pytest
import torch

from tokenweave_b200 import LLM, SamplingParams
from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
from tokenweave_b200.models.loader import save_hf_checkpoint

from tw_testing import hf_config_dict, make_hf_state, naive_logits


def _engine(path_or_name, **kw):
    args = dict(dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=512)
    args.update(kw)
    return LLM(path_or_name, **args)


def _runner(llm):
    return llm.llm_engine.core.executor.worker.runner


def _prompts(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def test_prompt_logprobs_match_the_naive_model(tmp_path):
    """Chunked prefill (3 chunks) with the prefix cache on: every prompt position still gets its entry, and a
    second request with the same prompt (a would-be cache hit) gets the same numbers."""
    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    st = make_hf_state(cfg, seed=2)
    save_hf_checkpoint(st, hf_config_dict(cfg), str(tmp_path))
    llm = _engine(str(tmp_path), max_num_batched_tokens=64, enable_prefix_caching=True)
    prompts = _prompts(cfg.vocab_size, [150, 20])
    sp = SamplingParams(temperature=0, max_tokens=2, prompt_logprobs=3)
    outs = llm.generate(prompts + [prompts[0]], [sp, SamplingParams(temperature=0, max_tokens=2), sp])
    assert outs[1].prompt_logprobs is None
    want = torch.log_softmax(naive_logits(cfg, st, prompts[0]), -1)
    for out in (outs[0], outs[2]):
        plp = out.prompt_logprobs
        assert len(plp) == 150 and plp[0] is None
        for p in range(1, 150):
            tok = prompts[0][p]
            assert abs(plp[p][tok] - want[p - 1, tok].item()) < 2e-4
            top = want[p - 1].topk(3)
            assert set(top.indices.tolist()) <= set(plp[p]) and len(plp[p]) <= 4
            for t, v in zip(top.indices.tolist(), top.values.tolist()):
                assert abs(plp[p][t] - v) < 2e-4
    llm.shutdown()


def test_phi3_packed_checkpoint_and_mistral_config(tmp_path):
    """Phi-3 stores the fused qkv / gate_up tensors; Mistral brings a sliding window and (newer configs) the
    rope settings under ``rope_parameters``. Both must load into the shared decoder and match the naive model."""
    preset = dict(MODEL_PRESETS["tiny-llama"], architecture="phi3", rope_theta=10000.0)
    cfg = ModelConfig(name="tiny-phi3", **preset)
    st = make_hf_state(cfg, seed=4)
    packed = {k: v for k, v in st.items() if not any(s in k for s in ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj"))}
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        packed[p + "self_attn.qkv_proj.weight"] = torch.cat([st[p + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0)
        packed[p + "mlp.gate_up_proj.weight"] = torch.cat([st[p + "mlp.gate_proj.weight"], st[p + "mlp.up_proj.weight"]], 0)
    save_hf_checkpoint(packed, hf_config_dict(cfg), str(tmp_path / "phi3"))
    prompts = _prompts(cfg.vocab_size, [40, 9])
    llm = _engine(str(tmp_path / "phi3"))
    assert llm.llm_engine.config.model.architecture == "phi3"
    r = _runner(llm)
    r.capture_logits = True
    llm.generate(prompts, SamplingParams(temperature=0, max_tokens=1))
    got = {rid: row for reqs, logits in r.captured_logits for rid, row in zip(reqs, logits)}
    for i, p in enumerate(prompts):
        torch.testing.assert_close(got[str(i)], naive_logits(cfg, st, p)[-1], atol=2e-4, rtol=2e-4)
    llm.shutdown()

    # a window (24 keys) shorter than the prompts, and a soft cap on the scores: prefill in chunks, then decode
    mcfg = ModelConfig(name="tiny-mistral", **dict(MODEL_PRESETS["tiny-llama"], architecture="mistral", rope_theta=1e6,
                                                   sliding_window=24, attn_logit_softcapping=5.0))
    hf = hf_config_dict(mcfg)
    del hf["rope_theta"]
    hf.update(rope_parameters={"rope_type": "default", "rope_theta": 1e6}, max_position_embeddings=2048)
    mst = make_hf_state(mcfg, seed=6)
    save_hf_checkpoint(mst, hf, str(tmp_path / "mistral"))
    llm = _engine(str(tmp_path / "mistral"), max_num_batched_tokens=32)
    m = llm.llm_engine.config.model
    assert (m.architecture, m.rope_theta, m.max_model_len, m.sliding_window, m.attn_logit_softcapping) == \
        ("mistral", 1e6, 2048, 24, 5.0)
    r = _runner(llm)
    r.capture_logits = True
    prompts = _prompts(mcfg.vocab_size, [70, 9])
    outs = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=3))
    first = {}
    for reqs, logits in r.captured_logits:
        for rid, row in zip(reqs, logits):
            first.setdefault(rid, row)
    for i, p in enumerate(prompts):
        torch.testing.assert_close(first[outs[i].request_id], naive_logits(mcfg, mst, p)[-1], atol=2e-4, rtol=2e-4)
        seq = list(p)
        for _ in range(3):
            seq.append(int(naive_logits(mcfg, mst, seq)[-1].argmax()))
        assert outs[i].outputs[0].token_ids == seq[len(p):]
    # the window matters for this prompt: full attention gives other logits
    full = ModelConfig(name="x", **dict(MODEL_PRESETS["tiny-llama"], architecture="mistral", rope_theta=1e6))
    assert (naive_logits(full, mst, prompts[0])[-1] - first[outs[0].request_id]).abs().max() > 1e-3
    llm.shutdown()


@pytest.mark.parametrize("arch", ["tiny-llama", "tiny-qwen2", "tiny-mixtral", "tiny-qwen3"])
def test_engine_matches_naive_forward(tmp_path, arch):
    preset = dict(MODEL_PRESETS[arch])
    if arch != "tiny-llama":
        preset.update(hidden_size=128, head_dim=32, intermediate_size=96, vocab_size=300, max_model_len=512)
    cfg = ModelConfig(name=arch, **preset)
    st = make_hf_state(cfg, seed=1)
    save_hf_checkpoint(st, hf_config_dict(cfg), str(tmp_path), shards=2)
    llm = _engine(str(tmp_path), max_num_batched_tokens=64)      # forces chunked prefill of the long prompt
    r = _runner(llm)
    r.capture_logits = True
    prompts = _prompts(cfg.vocab_size, [100, 7, 33])
    outs = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=3))
    # first logits of every request = logits at the last prompt position of the naive forward
    first = {}
    for reqs, logits in r.captured_logits:
        for rid, row in zip(reqs, logits):
            first.setdefault(rid, row)
    for i, p in enumerate(prompts):
        ref = naive_logits(cfg, st, p)[-1]
        torch.testing.assert_close(first[str(i)], ref, atol=2e-4, rtol=2e-4)
    # greedy continuation equals the naive model's
    for i, p in enumerate(prompts):
        seq = list(p)
        for _ in range(3):
            seq.append(int(naive_logits(cfg, st, seq)[-1].argmax()))
        assert outs[i].outputs[0].token_ids == seq[len(p):]


def test_split_path_equals_unsplit_path():
    """Tiny Llama-style decoder, fp32, 4 prompts of 64 tokens, greedy 16 tokens: the two-subset schedule
    must reproduce the unsplit path."""
    prompts = _prompts(1024, [64] * 4, seed=0)
    sp = SamplingParams(temperature=0, max_tokens=16)
    results = {}
    for name, kw in (("unsplit", dict(tokenweave_mode="fuse_only")),
                     ("split", dict(tokenweave_mode="overlap", tokenweave_force_overlap=True, tokenweave_threshold=128)),
                     ("split_off", dict(tokenweave_mode="overlap", tokenweave_force_overlap=True, tokenweave_threshold=128,
                                        tokenweave_split_offset=32))):
        llm = _engine("tiny-llama", seed=0, **kw)
        r = _runner(llm)
        r.capture_logits = True
        outs = llm.generate(prompts, sp)
        plan = r.planner.plan(256)
        assert plan.overlap == (name != "unsplit")
        if name == "split_off":
            assert plan.split == 160        # the cut falls inside the third prompt: a straddling request
        results[name] = ([o.outputs[0].token_ids for o in outs], torch.cat([l for _, l in r.captured_logits]))
        llm.shutdown()
    for name in ("split", "split_off"):
        assert results[name][0] == results["unsplit"][0]
        torch.testing.assert_close(results[name][1], results["unsplit"][1], atol=1e-5, rtol=1e-5)


def test_sampling_seeded_and_n():
    llm = _engine("tiny-llama")
    p = _prompts(1024, [20])
    sp = SamplingParams(temperature=0.8, top_p=0.9, top_k=50, max_tokens=8, seed=7, n=2, logprobs=2)
    a = llm.generate(p, sp)[0]
    b = llm.generate(p, sp)[0]
    assert [c.token_ids for c in a.outputs] == [c.token_ids for c in b.outputs]
    assert len(a.outputs) == 2 and a.outputs[0].token_ids != a.outputs[1].token_ids
    assert len(a.outputs[0].logprobs) == 8 and a.outputs[0].cumulative_logprob < 0


def test_text_prompt_and_stop_string():
    llm = LLM("tiny-llama", dtype="float32", device="cpu", tokenizer="byte", block_size=16, max_num_batched_tokens=256)
    out = llm.generate("hello world", SamplingParams(temperature=0, max_tokens=12))[0]
    assert out.prompt == "hello world" and len(out.outputs[0].token_ids) == 12
    assert isinstance(out.outputs[0].text, str)


def test_preemption_recompute_keeps_outputs():
    """With a KV pool too small for both requests one is preempted and recomputed; results must not change."""
    prompts = _prompts(1024, [60, 50], seed=3)
    sp = SamplingParams(temperature=0, max_tokens=24)
    big = _engine("tiny-llama", num_gpu_blocks_override=64)
    expect = [o.outputs[0].token_ids for o in big.generate(prompts, sp)]
    small = _engine("tiny-llama", num_gpu_blocks_override=10)     # 9 usable blocks = 144 tokens < 60+50+48
    got = [o.outputs[0].token_ids for o in small.generate(prompts, sp)]
    assert got == expect


def test_fp8_quantised_model_tracks_the_full_precision_model():
    """quantization="fp8" / "int8": every decoder linear runs on 8-bit weights (per-channel scales) and per-token
    quantised activations; logits stay close to the unquantised model's and greedy tokens mostly agree."""
    from tokenweave_b200.layers.linear import _QuantizableLinear
    prompts = _prompts(MODEL_PRESETS["tiny-llama"]["vocab_size"], [48, 9])
    logits = {}
    for quant in (None, "fp8", "int8"):
        llm = _engine("tiny-llama", quantization=quant, seed=3)
        r = _runner(llm)
        r.capture_logits = True
        llm.generate(prompts, SamplingParams(temperature=0, max_tokens=1))
        logits[quant] = torch.cat([lg for _, lg in r.captured_logits]).float()
        n_q = sum(1 for m in r.model.modules() if isinstance(m, _QuantizableLinear) and m.weight_scale is not None)
        assert (n_q > 0) == (quant is not None)
        if quant is not None:
            want = torch.float8_e4m3fn if quant == "fp8" else torch.int8
            assert all(m.weight.dtype == want for m in r.model.modules()
                       if isinstance(m, _QuantizableLinear) and m.weight_scale is not None)
    for quant in ("fp8", "int8"):
        cos = torch.nn.functional.cosine_similarity(logits[None], logits[quant], dim=-1)
        assert cos.min() > 0.98, (quant, cos)
    with pytest.raises(ValueError):
        _engine("tiny-llama", quantization="int3")


def test_fp8_checkpoint_loads_and_matches_online_quantisation(tmp_path):
    """A checkpoint that stores e4m3 weights with per-channel scales (plus static activation scales, which are
    ignored) runs on the fp8 path without a flag and gives what quantising the original weights online gives."""
    from tokenweave_b200.ops import reference as ref
    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    st = make_hf_state(cfg, seed=12)
    plain, quant = str(tmp_path / "plain"), str(tmp_path / "fp8")
    save_hf_checkpoint(st, hf_config_dict(cfg), plain)
    q_state = {}
    for name, t in st.items():
        if name.endswith("_proj.weight"):
            q, s = ref.quant_fp8(t)
            q_state[name] = q
            q_state[name[: -len(".weight")] + ".weight_scale"] = s.reshape(-1, 1)
            q_state[name[: -len(".weight")] + ".input_scale"] = torch.tensor(1.0)
        else:
            q_state[name] = t
    hf = hf_config_dict(cfg)
    hf["quantization_config"] = {"quant_method": "fp8", "activation_scheme": "static"}
    save_hf_checkpoint(q_state, hf, quant)
    prompts = _prompts(cfg.vocab_size, [60, 9])
    logits = []
    for path, kw in ((quant, {}), (plain, {"quantization": "fp8"})):
        llm = _engine(path, **kw)
        assert llm.llm_engine.config.quantization == "fp8"
        r = _runner(llm)
        r.capture_logits = True
        llm.generate(prompts, SamplingParams(temperature=0, max_tokens=1))
        got = {rid: row for reqs, lg in r.captured_logits for rid, row in zip(reqs, lg)}
        logits.append(torch.stack([got[str(i)] for i in range(len(prompts))]))
        llm.shutdown()
    torch.testing.assert_close(logits[0], logits[1], atol=1e-4, rtol=1e-4)
    bad = dict(hf_config_dict(cfg), quantization_config={"quant_method": "aqlm", "bits": 2})
    save_hf_checkpoint(st, bad, str(tmp_path / "aqlm"))
    with pytest.raises(ValueError, match="checkpoints are served"):
        _engine(str(tmp_path / "aqlm"))
