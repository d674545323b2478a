"""Pipeline parallelism on CPU (gloo): the layers are cut into stages, each stage a tensor-parallel group;
activations cross the cut by point-to-point sends. Tokens and first-token logits must equal the naive model's,
with chunked prefill, the token-split schedule and a prefix cache in play."""
import pytest
import torch

from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
from tokenweave_b200.models.loader import save_hf_checkpoint

from tw_testing import hf_config_dict, make_hf_state, naive_logits, run_ranks


def _rank(rank, world, ckpt, tp, pp, prompts, expect_path):
    from tokenweave_b200 import LLM, SamplingParams
    from tokenweave_b200.parallel.state import get_tp
    llm = LLM(ckpt, dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=96,
              tensor_parallel_size=tp, pipeline_parallel_size=pp, distributed_executor_backend="external_launcher",
              tokenweave_threshold=64, enable_prefix_caching=True)
    st = get_tp()
    assert (st.world_size, st.pp_size, st.rank, st.pp_rank) == (tp, pp, rank % tp, rank // tp)
    model = llm.llm_engine.core.executor.worker.runner.model
    assert len(model.layers) < model.cfg.num_layers and (model.boundary_norm_w is None) == st.is_last_stage
    r = llm.llm_engine.core.executor.worker.runner
    r.capture_logits = True
    expect = torch.load(expect_path)
    for _ in range(2):                     # the second pass hits the prefix cache on every stage
        r.captured_logits = []
        outs = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=4, ignore_eos=True))
        assert [o.outputs[0].token_ids for o in outs] == expect["tokens"]
        if st.is_last_stage:
            first = {}
            for reqs, logits in r.captured_logits:
                for rid, row in zip(reqs, logits):
                    first.setdefault(rid, row)
            got = torch.stack([first[o.request_id] for o in outs])
            torch.testing.assert_close(got, expect["logits"], atol=3e-4, rtol=3e-4)
        else:
            assert r.captured_logits == []          # inner stages never see logits
    llm.shutdown()


@pytest.mark.parametrize("tp,pp", [(1, 2), (2, 2), (1, 3)])
def test_pipeline_stages_match_the_naive_model(tmp_path, tp, pp):
    cfg = ModelConfig(name="tiny-llama", **dict(MODEL_PRESETS["tiny-llama"], num_layers=3))
    st = make_hf_state(cfg, seed=21)
    ckpt = str(tmp_path / "ckpt")
    save_hf_checkpoint(st, hf_config_dict(cfg), ckpt)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (150, 20, 70)]
    tokens, logits = [], []
    for p in prompts:
        seq = list(p)
        logits.append(naive_logits(cfg, st, seq)[-1])
        for _ in range(4):
            seq.append(int(naive_logits(cfg, st, seq)[-1].argmax()))
        tokens.append(seq[len(p):])
    ep = str(tmp_path / "expect.pt")
    torch.save({"tokens": tokens, "logits": torch.stack(logits)}, ep)
    run_ranks(_rank, tp * pp, ckpt, tp, pp, prompts, ep)


def test_pipeline_stages_under_the_multiprocess_executor(tmp_path):
    """The engine process spawns tp x pp workers; rank 0 (an inner stage) answers with the broadcast result."""
    from tokenweave_b200 import LLM, SamplingParams
    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    st = make_hf_state(cfg, seed=22)
    ckpt = str(tmp_path / "ckpt")
    save_hf_checkpoint(st, hf_config_dict(cfg), ckpt)
    prompt = list(range(3, 60))
    seq = list(prompt)
    for _ in range(5):
        seq.append(int(naive_logits(cfg, st, seq)[-1].argmax()))
    llm = LLM(ckpt, dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=64,
              tensor_parallel_size=1, pipeline_parallel_size=2, distributed_executor_backend="mp")
    try:
        out = llm.generate([prompt], SamplingParams(temperature=0, max_tokens=5, ignore_eos=True, logprobs=1))[0]
        assert out.outputs[0].token_ids == seq[len(prompt):]
        assert len(out.outputs[0].logprobs) == 5          # log-probabilities travel back from the last stage too
    finally:
        llm.shutdown()


def _sharded_rank(rank, world, ckpt, out_dir, prompt, expect):
    from tokenweave_b200 import LLM, SamplingParams
    sp = SamplingParams(temperature=0, max_tokens=4, ignore_eos=True)
    common = dict(dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=64,
                  tensor_parallel_size=2, distributed_executor_backend="external_launcher")
    llm = LLM(ckpt, **common)
    llm.save_sharded_state(out_dir)
    assert llm.generate([prompt], sp)[0].outputs[0].token_ids == expect
    # the same job starts again from the per-rank files: no HuggingFace tensors are read
    import torch.distributed as dist
    dist.barrier()
    from tokenweave_b200.models.loader import load_model_weights
    model = llm.llm_engine.core.executor.worker.runner.model
    for p_ in model.parameters():
        p_.data.zero_()
    cfg2 = llm.llm_engine.config
    cfg2.load_format, cfg2.model.path = "sharded_state", out_dir
    load_model_weights(model, cfg2)
    assert llm.generate([prompt], sp)[0].outputs[0].token_ids == expect
    llm.shutdown()


def test_sharded_state_round_trip_under_tp2(tmp_path):
    """``LLM.save_sharded_state`` writes every rank's parameters; ``load_format="sharded_state"`` reads them back."""
    import os
    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    st = make_hf_state(cfg, seed=23)
    ckpt, out_dir = str(tmp_path / "ckpt"), str(tmp_path / "sharded")
    save_hf_checkpoint(st, hf_config_dict(cfg), ckpt)
    prompt = list(range(9, 50))
    seq = list(prompt)
    for _ in range(4):
        seq.append(int(naive_logits(cfg, st, seq)[-1].argmax()))
    run_ranks(_sharded_rank, 2, ckpt, out_dir, prompt, seq[len(prompt):])
    assert {"rank_0.safetensors", "rank_1.safetensors", "config.json"} <= set(os.listdir(out_dir))
    # a fresh single-rank engine on a two-rank dump must be refused, not mis-loaded
    from tokenweave_b200 import LLM
    with pytest.raises(ValueError, match="shape"):
        LLM(out_dir, dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, load_format="sharded_state")
