"""LoRA serving on CPU (fp32): a request served through an adapter must see exactly the model whose weights
are ``W + (alpha / r) B A``; requests with different adapters (and without any) share a batch; TP=2 over gloo
shards the adapter like the base layers."""
import json
import os

import torch

from tokenweave_b200 import LLM, SamplingParams
from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
from tokenweave_b200.lora import LoRARequest
from tokenweave_b200.models.loader import save_hf_checkpoint

from tw_testing import hf_config_dict, make_hf_state, naive_logits, run_ranks

TARGETS = {"q_proj": "self_attn", "k_proj": "self_attn", "v_proj": "self_attn", "o_proj": "self_attn",
           "gate_proj": "mlp", "up_proj": "mlp", "down_proj": "mlp"}


def _make_adapter(path, cfg, state, r, alpha, seed, targets=tuple(TARGETS)):
    """Writes a PEFT-style adapter directory and returns the merged HuggingFace state dict."""
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    tensors, merged = {}, dict(state)
    for l in range(cfg.num_layers):
        for t in targets:
            name = f"model.layers.{l}.{TARGETS[t]}.{t}.weight"
            out_f, in_f = state[name].shape
            A = torch.randn(r, in_f, generator=g) * 0.05
            B = torch.randn(out_f, r, generator=g) * 0.05
            base = f"base_model.model.model.layers.{l}.{TARGETS[t]}.{t}"
            tensors[base + ".lora_A.weight"] = A
            tensors[base + ".lora_B.weight"] = B
            merged[name] = state[name] + (alpha / r) * (B @ A)
    os.makedirs(path, exist_ok=True)
    save_file(tensors, os.path.join(path, "adapter_model.safetensors"))
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"r": r, "lora_alpha": alpha, "target_modules": list(targets), "peft_type": "LORA"}, f)
    return merged


def _setup(tmp_path):
    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    st = make_hf_state(cfg, seed=11)
    ckpt = str(tmp_path / "base")
    save_hf_checkpoint(st, hf_config_dict(cfg), ckpt)
    m1 = _make_adapter(str(tmp_path / "ad1"), cfg, st, r=4, alpha=8, seed=1)
    m2 = _make_adapter(str(tmp_path / "ad2"), cfg, st, r=6, alpha=3, seed=2, targets=("q_proj", "v_proj", "down_proj"))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (150, 33, 90)]
    return cfg, st, ckpt, (m1, m2), prompts


def _first_logits(llm, prompts, loras):
    r = llm.llm_engine.core.executor.worker.runner
    r.capture_logits = True
    r.captured_logits = []
    outs = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=3), lora_request=loras)
    first = {}
    for reqs, logits in r.captured_logits:
        for rid, row in zip(reqs, logits):
            first.setdefault(rid, row)
    return [first[o.request_id] for o in outs], [o.outputs[0].token_ids for o in outs]


def test_mixed_adapters_in_one_batch_match_merged_weights(tmp_path):
    cfg, st, ckpt, (m1, m2), prompts = _setup(tmp_path)
    lr1 = LoRARequest("one", 1, str(tmp_path / "ad1"))
    lr2 = LoRARequest("two", 2, str(tmp_path / "ad2"))
    llm = LLM(ckpt, dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=128,
              enable_lora=True, enable_prefix_caching=True, tokenweave_force_overlap=True, tokenweave_threshold=64)
    logits, toks = _first_logits(llm, prompts, [lr1, None, lr2])
    for lg, p, state in zip(logits, prompts, (m1, st, m2)):
        torch.testing.assert_close(lg, naive_logits(cfg, state, p)[-1], atol=3e-4, rtol=3e-4)
    # the same prompt through another adapter must not reuse the first adapter's cached prefix
    logits2, _ = _first_logits(llm, [prompts[0], prompts[0]], [lr2, None])
    torch.testing.assert_close(logits2[0], naive_logits(cfg, m2, prompts[0])[-1], atol=3e-4, rtol=3e-4)
    torch.testing.assert_close(logits2[1], naive_logits(cfg, st, prompts[0])[-1], atol=3e-4, rtol=3e-4)
    # greedy continuation under adapter 1 equals the merged model's
    seq = list(prompts[0])
    for _ in range(3):
        seq.append(int(naive_logits(cfg, m1, seq)[-1].argmax()))
    assert toks[0] == seq[len(prompts[0]):]
    llm.shutdown()
    plain = LLM(ckpt, dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16)
    try:
        plain.generate([prompts[1]], SamplingParams(max_tokens=1), lora_request=lr1)
        raise AssertionError("a LoRA request without enable_lora must be refused")
    except ValueError:
        pass
    plain.shutdown()


def _tp_rank(rank, world, ckpt, ad1, prompts, expect_path):
    llm = LLM(ckpt, dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=256,
              enable_lora=True, tensor_parallel_size=world, distributed_executor_backend="external_launcher",
              tokenweave_threshold=128)
    logits, _ = _first_logits(llm, prompts, [LoRARequest("one", 1, ad1), None, LoRARequest("one", 1, ad1)])
    torch.testing.assert_close(torch.stack(logits), torch.load(expect_path), atol=3e-4, rtol=3e-4)
    llm.shutdown()


def test_lora_under_tp2(tmp_path):
    cfg, st, ckpt, (m1, _), prompts = _setup(tmp_path)
    expect = torch.stack([naive_logits(cfg, s, p)[-1] for s, p in zip((m1, st, m1), prompts)])
    ep = str(tmp_path / "expect.pt")
    torch.save(expect, ep)
    run_ranks(_tp_rank, 2, ckpt, str(tmp_path / "ad1"), prompts, ep)
