"""Rotary tables for the scaling variants (linear, dynamic NTK, YaRN, Llama-3) against the Hugging Face
initialisers, which the reference's rotary_embedding.py classes reproduce."""
import pytest
import torch

from tokenweave_b200.ops.reference import build_cos_sin_cache

D, THETA = 64, 10000.0


def _hf_table(kind, max_pos, cfg_max_pos, **extra):
    rope_utils = pytest.importorskip("transformers.modeling_rope_utils")
    from transformers import LlamaConfig
    try:
        cfg = LlamaConfig(hidden_size=D * 4, num_attention_heads=4, max_position_embeddings=cfg_max_pos,
                          rope_parameters=dict(rope_type=kind, rope_theta=THETA, **extra))
        fn = rope_utils.ROPE_INIT_FUNCTIONS[kind]
        inv, att = fn(cfg, "cpu", seq_len=max_pos) if kind == "dynamic" else fn(cfg, "cpu")
    except (TypeError, KeyError, AttributeError) as e:     # another transformers release, another config schema
        pytest.skip(f"transformers rope API differs: {e}")
    fr = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv.double())
    return (torch.cat([fr.cos(), fr.sin()], -1) * att).float()


@pytest.mark.parametrize("kind,extra,cfg_max_pos", [
    ("linear", dict(factor=2.0), 8192),
    ("yarn", dict(factor=4.0, original_max_position_embeddings=2048), 8192),
    ("yarn", dict(factor=8.0, original_max_position_embeddings=1024, beta_fast=16.0, beta_slow=2.0), 8192),
    ("llama3", dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=2048), 8192),
    ("dynamic", dict(factor=4.0), 2048),
])
def test_scaled_tables_match_hugging_face(kind, extra, cfg_max_pos):
    want = _hf_table(kind, 8192, cfg_max_pos, **extra)
    ours = dict(rope_type=kind, **extra)
    if kind == "dynamic":
        ours["original_max_position_embeddings"] = cfg_max_pos
    got = build_cos_sin_cache(D, 8192, THETA, ours)
    # the oracle keeps inv_freq in fp32; at position 8191 that is worth a few 1e-4 of phase
    torch.testing.assert_close(got, want, atol=1e-3, rtol=0)
    if kind == "yarn":
        assert got.abs().max() > 1.05           # the attention temperature sits in the table


def test_unknown_scaling_is_refused_and_default_is_plain():
    with pytest.raises(ValueError):
        build_cos_sin_cache(D, 16, THETA, dict(rope_type="longrope", factor=2.0))
    torch.testing.assert_close(build_cos_sin_cache(D, 16, THETA, dict(rope_type="default")),
                               build_cos_sin_cache(D, 16, THETA, None))
