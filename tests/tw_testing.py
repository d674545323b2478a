"""Shared helpers of the test-suite: a naive dense reference model in HuggingFace weight layout and a
launcher for multi-process (gloo) tests."""
import math
import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def make_hf_state(cfg, seed=0, dtype=torch.float32):
    """Random weights in HuggingFace naming for a ModelConfig (dense or Mixtral)."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(dtype)
    H, D = cfg.hidden_size, cfg.head_dim
    st = {"model.embed_tokens.weight": r(cfg.vocab_size, H), "model.norm.weight": (1 + 0.1 * torch.randn(H, generator=g)).to(dtype),
          "lm_head.weight": r(cfg.vocab_size, H)}
    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        st[p + "input_layernorm.weight"] = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
        st[p + "post_attention_layernorm.weight"] = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
        st[p + "self_attn.q_proj.weight"] = r(cfg.num_q_heads * D, H)
        st[p + "self_attn.k_proj.weight"] = r(cfg.num_kv_heads * D, H)
        st[p + "self_attn.v_proj.weight"] = r(cfg.num_kv_heads * D, H)
        st[p + "self_attn.o_proj.weight"] = r(H, cfg.num_q_heads * D)
        if cfg.qkv_bias:
            st[p + "self_attn.q_proj.bias"] = r(cfg.num_q_heads * D)
            st[p + "self_attn.k_proj.bias"] = r(cfg.num_kv_heads * D)
            st[p + "self_attn.v_proj.bias"] = r(cfg.num_kv_heads * D)
        if getattr(cfg, "qk_norm", False):
            st[p + "self_attn.q_norm.weight"] = (1 + 0.2 * torch.randn(D, generator=g)).to(dtype)
            st[p + "self_attn.k_norm.weight"] = (1 + 0.2 * torch.randn(D, generator=g)).to(dtype)
        if cfg.num_experts:
            st[p + "block_sparse_moe.gate.weight"] = r(cfg.num_experts, H)
            for e in range(cfg.num_experts):
                st[p + f"block_sparse_moe.experts.{e}.w1.weight"] = r(cfg.intermediate_size, H)
                st[p + f"block_sparse_moe.experts.{e}.w3.weight"] = r(cfg.intermediate_size, H)
                st[p + f"block_sparse_moe.experts.{e}.w2.weight"] = r(H, cfg.intermediate_size)
        else:
            st[p + "mlp.gate_proj.weight"] = r(cfg.intermediate_size, H)
            st[p + "mlp.up_proj.weight"] = r(cfg.intermediate_size, H)
            st[p + "mlp.down_proj.weight"] = r(H, cfg.intermediate_size)
    return st


def hf_config_dict(cfg):
    arch = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "mixtral": "MixtralForCausalLM",
            "qwen3": "Qwen3ForCausalLM", "mistral": "MistralForCausalLM", "phi3": "Phi3ForCausalLM"}[cfg.architecture]
    d = dict(architectures=[arch], hidden_size=cfg.hidden_size, num_hidden_layers=cfg.num_layers,
             num_attention_heads=cfg.num_q_heads, num_key_value_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
             intermediate_size=cfg.intermediate_size, vocab_size=cfg.vocab_size, rms_norm_eps=cfg.rms_norm_eps,
             rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_model_len, torch_dtype="float32",
             attention_bias=cfg.qkv_bias)
    if getattr(cfg, "sliding_window", 0):
        d["sliding_window"] = cfg.sliding_window
    if getattr(cfg, "attn_logit_softcapping", 0.0):
        d["attn_logit_softcapping"] = cfg.attn_logit_softcapping
    if cfg.num_experts:
        d.update(num_local_experts=cfg.num_experts, num_experts_per_tok=cfg.num_experts_per_tok)
    return d


def naive_logits(cfg, st, ids, cos_sin=None):
    """Dense fp32 forward of one sequence (no paging, no sharding): logits for every position. ``cos_sin``:
    optional ([T, D/2] cos, [T, D/2] sin) tables for rope variants; the default is plain rope."""
    x = st["model.embed_tokens.weight"].float()[ids]
    T, D, half = len(ids), cfg.head_dim, cfg.head_dim // 2
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, dtype=torch.float64) * 2 / D))
    fr = torch.outer(torch.arange(T, dtype=torch.float64), inv)
    cos, sin = fr.cos().float()[:, None, :], fr.sin().float()[:, None, :]
    if cos_sin is not None:
        cos, sin = cos_sin[0][:, None, :], cos_sin[1][:, None, :]

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w.float()

    def rope(t):
        a, b = t[..., :half], t[..., half:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    for l in range(cfg.num_layers):
        p = f"model.layers.{l}."
        h = norm(x, st[p + "input_layernorm.weight"])
        q = h @ st[p + "self_attn.q_proj.weight"].float().t()
        k = h @ st[p + "self_attn.k_proj.weight"].float().t()
        v = h @ st[p + "self_attn.v_proj.weight"].float().t()
        if cfg.qkv_bias:
            q, k, v = (q + st[p + "self_attn.q_proj.bias"].float(), k + st[p + "self_attn.k_proj.bias"].float(),
                       v + st[p + "self_attn.v_proj.bias"].float())
        q, k = q.view(T, cfg.num_q_heads, D), k.view(T, cfg.num_kv_heads, D)
        if getattr(cfg, "qk_norm", False):
            q, k = norm(q, st[p + "self_attn.q_norm.weight"]), norm(k, st[p + "self_attn.k_norm.weight"])
        q, k = rope(q), rope(k)
        v = v.view(T, cfg.num_kv_heads, D)
        rep = cfg.num_q_heads // cfg.num_kv_heads
        k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(D)
        cap = getattr(cfg, "attn_logit_softcapping", 0.0)
        if cap:
            s = cap * torch.tanh(s / cap)
        hidden_keys = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
        if getattr(cfg, "sliding_window", 0):
            hidden_keys |= torch.tril(torch.ones(T, T, dtype=torch.bool), -cfg.sliding_window)
        s = s.masked_fill(hidden_keys, float("-inf"))
        o = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(T, -1)
        x = x + o @ st[p + "self_attn.o_proj.weight"].float().t()
        h = norm(x, st[p + "post_attention_layernorm.weight"])
        if cfg.num_experts:
            logits = h @ st[p + "block_sparse_moe.gate.weight"].float().t()
            w, idx = logits.softmax(-1).topk(cfg.num_experts_per_tok, -1)
            w = w / w.sum(-1, keepdim=True)
            y = torch.zeros_like(h)
            for t in range(T):
                for j in range(cfg.num_experts_per_tok):
                    e = int(idx[t, j])
                    pe = p + f"block_sparse_moe.experts.{e}."
                    a = F.silu(h[t] @ st[pe + "w1.weight"].float().t()) * (h[t] @ st[pe + "w3.weight"].float().t())
                    y[t] += w[t, j] * (a @ st[pe + "w2.weight"].float().t())
            x = x + y
        else:
            a = F.silu(h @ st[p + "mlp.gate_proj.weight"].float().t()) * (h @ st[p + "mlp.up_proj.weight"].float().t())
            x = x + a @ st[p + "mlp.down_proj.weight"].float().t()
    return norm(x, st["model.norm.weight"]) @ st["lm_head.weight"].float().t()


def _entry(rank, world, port, fn, args, errq):
    try:
        os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                          MASTER_PORT=str(port))
        sys.path.insert(0, ROOT)
        torch.set_num_threads(2)
        fn(rank, world, *args)
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_ranks(fn, world, *args, timeout=240):
    """Run ``fn(rank, world, *args)`` in ``world`` spawned processes; raises if any rank fails."""
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    failed = []
    for r, p in enumerate(procs):
        if p.is_alive():
            p.terminate()
            failed.append(f"rank {r} timed out")
        elif p.exitcode != 0:
            failed.append(f"rank {r} exit code {p.exitcode}")
    msgs = []
    while not errq.empty():
        msgs.append("rank %d:\n%s" % errq.get())
    assert not failed, "; ".join(failed) + "\n" + "\n".join(msgs)
