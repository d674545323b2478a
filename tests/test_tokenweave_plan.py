"""TokenWeave config files, split planner and split metadata."""
import json

from tokenweave_b200.tokenweave.config import CONFIG_DIR, TokenWeavePlanner, load_config
from tokenweave_b200.worker.split_metadata import split_batch
from tokenweave_b200.layers.attention import plan_attention


def test_shipped_configs_have_reference_schema():
    files = sorted(CONFIG_DIR.glob("*_config_*.json"))
    assert {f.name for f in files} >= {"llama_config_8.json", "llama_config_4.json", "qwen2_config_8.json",
                                       "qwen2_config_4.json", "mixtral_config_8.json"}
    for f in files:
        cfg = load_config(str(f))
        assert all(isinstance(k, int) for k in cfg)
        for v in cfg.values():
            assert {"attention_ctas", "mlp_ctas", "split_offset"} <= set(v)


def test_nearest_key_and_split_formula(tmp_path):
    p = tmp_path / "c.json"
    p.write_text(json.dumps({"1024": {"attention_ctas": 4, "mlp_ctas": 2, "split_offset": 0},
                             "8192": {"attention_ctas": 8, "mlp_ctas": 4, "split_offset": 256}}))
    pl = TokenWeavePlanner("llama", 8, "overlap", str(p))
    a = pl.plan(7000)         # nearest key 8192
    assert a.overlap and a.padded_tokens == 7168 and a.split == 7168 // 2 + 256
    assert (a.attention_ctas, a.mlp_ctas) == (8, 4)
    b = pl.plan(1500)         # nearest key 1024
    assert b.overlap and b.padded_tokens == 1536 and b.split == 768 and b.attention_ctas == 4
    c = pl.plan(1000)         # below the llama threshold: fuse-only, padded to the TP size
    assert not c.overlap and c.padded_tokens == 1000
    d = pl.plan(1001)
    assert d.padded_tokens == 1008
    assert TokenWeavePlanner("mixtral", 8, "overlap", str(p)).plan(1500).overlap is False   # threshold 2048


def test_split_divisible_by_world_and_env_override(monkeypatch):
    pl = TokenWeavePlanner("llama", 8, "overlap")
    # the tuned B200 file marks the 1024-token entry "overlap": 0 (the unsplit fused schedule measured faster)
    assert pl.plan(1024).overlap is False and pl.plan(1535).overlap is False and pl.plan(1537).overlap is True
    forced = TokenWeavePlanner("llama", 8, "overlap", force_overlap=True)
    for t in (1024, 1025, 3000, 8192, 12345):
        p = forced.plan(t)
        assert p.overlap and p.split % 8 == 0 and (p.padded_tokens - p.split) % 8 == 0
        assert p.tokens_0 + p.tokens_1 == t
    monkeypatch.setenv("TW_SPLIT_OFFSET", "128")
    assert pl.plan(4096).split == 2048 + 128
    assert TokenWeavePlanner("llama", 1, "overlap").plan(4096).overlap is False
    assert TokenWeavePlanner("llama", 1, "overlap", force_overlap=True).plan(4096).overlap is True


def test_split_batch_straddling_request():
    q_lens, kv_lens = [100, 300, 50], [100, 900, 50]
    first, second = split_batch(q_lens, kv_lens, 256)
    assert first == [(0, 100, 100), (1, 156, 900 - 144)]
    assert second == [(1, 144, 900), (2, 50, 50)]
    first, second = split_batch(q_lens, kv_lens, 400)   # cut on a request boundary: nobody is shared
    assert first == [(0, 100, 100), (1, 300, 900)] and second == [(2, 50, 50)]
    first, second = split_batch([10], [10], 256)
    assert first == [(0, 10, 10)] and second == []


def test_plan_attention_routing():
    tile_seq, tile_q0, tok_row, tok_seq, tok_kv = plan_attention([300, 1, 5, 128], [300, 77, 40, 640])
    assert sorted(zip(tile_seq, tile_q0)) == [(0, 0), (0, 128), (0, 256), (3, 0)]
    assert (tile_seq[0], tile_q0[0]) == (3, 0)            # longest causal span first
    assert tok_row == [300, 301, 302, 303, 304, 305] and tok_seq == [1, 2, 2, 2, 2, 2]
    assert tok_kv == [77, 36, 37, 38, 39, 40]
    # a decode-only step takes the loop-free path and must say what the loop says for it
    tile_seq, tile_q0, tok_row, tok_seq, tok_kv = plan_attention([1, 1, 1], [9, 300, 41])
    assert list(tile_seq) == [] and list(tile_q0) == []
    assert list(tok_row) == [0, 1, 2] and list(tok_seq) == [0, 1, 2] and list(tok_kv) == [9, 300, 41]
    # one two-token row (a verified draft) in the batch: back to the general path
    _, _, tok_row, tok_seq, tok_kv = plan_attention([1, 2], [9, 31])
    assert list(tok_row) == [0, 1, 2] and list(tok_seq) == [0, 1, 1] and list(tok_kv) == [9, 30, 31]
