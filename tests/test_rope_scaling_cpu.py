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
        build_cos_sin_cache(D, 16, THETA, dict(rope_type="mrope", factor=2.0))
    with pytest.raises(ValueError):
        build_cos_sin_cache(D, 16, THETA, dict(rope_type="longrope", factor=2.0))      # no factor lists
    torch.testing.assert_close(build_cos_sin_cache(D, 16, THETA, dict(rope_type="default")),
                               build_cos_sin_cache(D, 16, THETA, None))


def test_longrope_tables_and_the_position_shift():
    """Phi-3 LongRoPE: short-factor rows for contexts inside the original window, long-factor rows behind them;
    a step that reaches beyond the window reads the long rows (checked through the engine against a naive model
    that uses the long factors for all its tokens)."""
    rope_utils = pytest.importorskip("transformers.modeling_rope_utils")
    from transformers import Phi3Config
    from tokenweave_b200.ops.reference import longrope_offset
    half = D // 2
    g = torch.Generator().manual_seed(0)
    short = (1 + torch.rand(half, generator=g)).tolist()
    long_ = (1 + 4 * torch.rand(half, generator=g)).tolist()
    rs = dict(rope_type="longrope", short_factor=short, long_factor=long_, original_max_position_embeddings=256)
    table = build_cos_sin_cache(D, 1024, THETA, rs)
    assert table.shape == (256 + 1024, D) and longrope_offset(rs, 1024) == 256 and longrope_offset(None, 1024) == 0
    try:
        cfg = Phi3Config(hidden_size=D * 4, num_attention_heads=4, max_position_embeddings=1024,
                         original_max_position_embeddings=256, rope_parameters=dict(rope_theta=THETA, **rs))
        for seq_len, rows in ((100, slice(0, 256)), (1000, slice(256, 1280))):
            inv, att = rope_utils.ROPE_INIT_FUNCTIONS["longrope"](cfg, "cpu", seq_len=seq_len)
            n = rows.stop - rows.start
            fr = torch.outer(torch.arange(n, dtype=torch.float64), inv.double())
            want = (torch.cat([fr.cos(), fr.sin()], -1) * att).float()
            torch.testing.assert_close(table[rows], want, atol=1e-3, rtol=0)
    except (TypeError, KeyError, AttributeError) as e:
        pytest.skip(f"transformers rope API differs: {e}")


def test_longrope_engine_uses_long_factors_beyond_the_window(tmp_path):
    import math
    from tokenweave_b200 import LLM, SamplingParams
    from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
    from tokenweave_b200.models.loader import save_hf_checkpoint
    from tw_testing import hf_config_dict, make_hf_state, naive_logits
    half = 32
    g = torch.Generator().manual_seed(1)
    rs = dict(rope_type="longrope", short_factor=(1 + torch.rand(half, generator=g)).tolist(),
              long_factor=(1 + 3 * torch.rand(half, generator=g)).tolist(), original_max_position_embeddings=64)
    cfg = ModelConfig(name="tiny-phi3", **dict(MODEL_PRESETS["tiny-llama"], architecture="phi3", rope_theta=THETA,
                                               max_model_len=512, rope_scaling=rs))
    st = make_hf_state(cfg, seed=3)
    hf = hf_config_dict(cfg)
    hf["rope_scaling"] = rs
    save_hf_checkpoint(st, hf, str(tmp_path))
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16,
              max_num_batched_tokens=256)
    r = llm.llm_engine.core.executor.worker.runner
    r.capture_logits = True
    prompts = [list(range(3, 40)), list(range(5, 150))]           # inside the window / beyond it
    got = []
    for p in prompts:                                             # one at a time: the shift is per step
        r.captured_logits = []
        llm.generate([p], SamplingParams(temperature=0, max_tokens=1))
        got.append(r.captured_logits[0][1][0])
    llm.shutdown()

    def naive(p, factors):
        """The naive model with per-frequency factors folded into an equivalent theta-free table."""
        import tw_testing
        mscale = math.sqrt(1 + math.log(512 / 64) / math.log(64))
        Dh = cfg.head_dim
        inv = 1.0 / (THETA ** (torch.arange(0, Dh // 2, dtype=torch.float64) * 2 / Dh)) / torch.tensor(factors, dtype=torch.float64)
        fr = torch.outer(torch.arange(len(p), dtype=torch.float64), inv)
        return tw_testing.naive_logits(cfg, st, p, cos_sin=((fr.cos() * mscale).float(), (fr.sin() * mscale).float()))[-1]
    torch.testing.assert_close(got[0], naive(prompts[0], rs["short_factor"]), atol=3e-4, rtol=3e-4)
    torch.testing.assert_close(got[1], naive(prompts[1], rs["long_factor"]), atol=3e-4, rtol=3e-4)
