"""GPU runs of the parallel paths the tensor-parallel suite does not reach: pipeline stages (1 x 2) and LoRA
adapters under tensor parallelism on two GPUs, and the KV-transfer connector between two engines whose caches
live in GPU memory (one GPU). The vocabulary-parallel embedding rides on the tensor-parallel suite
(test_tp_gpu.py, modes ending in ``+vpe``)."""
import os

import pytest
import torch

from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
from tokenweave_b200.models.loader import save_hf_checkpoint

from tw_testing import hf_config_dict, make_hf_state, naive_logits, run_ranks

pytestmark = pytest.mark.gpu

ARCH = "tiny-llama-d128"


def _checkpoint(tmp_path, seed):
    cfg = ModelConfig(name=ARCH, **MODEL_PRESETS[ARCH])
    st = make_hf_state(cfg, seed=seed)
    hf = hf_config_dict(cfg)
    hf["torch_dtype"] = "bfloat16"
    ckpt = str(tmp_path / "base")
    save_hf_checkpoint({k: v.to(torch.bfloat16) for k, v in st.items()}, hf, ckpt)
    return cfg, {k: v.to(torch.bfloat16).float() for k, v in st.items()}, ckpt      # what the engine holds


def _prompts(cfg, lens):
    g = torch.Generator().manual_seed(0)
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]


def _first_rows(runner, outs):
    first = {}
    for reqs, logits in runner.captured_logits:
        for rid, row in zip(reqs, logits):
            first.setdefault(rid, row)
    return torch.stack([first[o.request_id] for o in outs])


# ---- pipeline parallelism: two stages, one GPU each ------------------------------------------------------------
def _pp_rank(rank, world, ckpt, prompts, expect_path):
    from tokenweave_b200 import LLM, SamplingParams, ops
    from tokenweave_b200.parallel.state import get_tp
    llm = LLM(ckpt, device="cuda", skip_tokenizer_init=True, block_size=128, max_num_batched_tokens=512,
              num_gpu_blocks_override=64, tensor_parallel_size=1, pipeline_parallel_size=world,
              distributed_executor_backend="external_launcher")
    st = get_tp()
    assert (st.world_size, st.pp_size, st.pp_rank) == (1, world, rank)
    runner = llm.llm_engine.core.executor.worker.runner
    runner.capture_logits = True
    outs = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=4, ignore_eos=True))
    torch.cuda.synchronize()
    ops.check_status()
    expect = torch.load(expect_path)
    # every stage learns the sampled tokens; the same kernels ran on the same data as on one GPU
    assert [o.outputs[0].token_ids for o in outs] == expect["tokens"]
    if st.is_last_stage:
        got = _first_rows(runner, outs).float().cpu()
        torch.testing.assert_close(got, expect["logits"], atol=2e-2, rtol=2e-2)
    else:
        assert runner.captured_logits == []
    llm.shutdown()


def test_pipeline_two_stages_match_one_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from tokenweave_b200 import LLM, SamplingParams
    cfg, _, ckpt = _checkpoint(tmp_path, seed=41)
    prompts = _prompts(cfg, [700, 90, 333])          # 700 tokens: chunked prefill over two steps of 512
    llm = LLM(ckpt, device="cuda", skip_tokenizer_init=True, block_size=128, max_num_batched_tokens=512,
              num_gpu_blocks_override=64)
    runner = llm.llm_engine.core.executor.worker.runner
    runner.capture_logits = True
    outs = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=4, ignore_eos=True))
    ep = str(tmp_path / "expect.pt")
    torch.save({"tokens": [o.outputs[0].token_ids for o in outs], "logits": _first_rows(runner, outs).float().cpu()}, ep)
    llm.shutdown()
    run_ranks(_pp_rank, 2, ckpt, prompts, ep, timeout=300)


# ---- LoRA adapters with the base weights sharded over two GPUs -------------------------------------------------
def _lora_rank(rank, world, ckpt, ad1, ad2, prompts, expect_path):
    from tokenweave_b200 import LLM, ops
    from tokenweave_b200.lora import LoRARequest
    from test_lora_cpu import _first_logits
    llm = LLM(ckpt, device="cuda", skip_tokenizer_init=True, block_size=128, max_num_batched_tokens=1024,
              num_gpu_blocks_override=64, enable_lora=True, tensor_parallel_size=world,
              distributed_executor_backend="external_launcher", tokenweave_threshold=256)
    logits, _ = _first_logits(llm, prompts, [LoRARequest("one", 1, ad1), None, LoRARequest("two", 2, ad2)])
    torch.cuda.synchronize()
    ops.check_status()
    expect = torch.load(expect_path)
    for lg, want, wrong in zip(logits, expect["want"], expect["wrong"]):
        err = (lg.float().cpu() - want).abs().max().item()
        assert err < 0.08 * max(1.0, want.abs().max().item()), err
        assert err < (lg.float().cpu() - wrong).abs().max().item()      # the adapter's model, not the other one
    llm.shutdown()


def test_lora_under_tensor_parallelism(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from test_lora_cpu import _make_adapter
    cfg, st, ckpt = _checkpoint(tmp_path, seed=5)
    ad1, ad2 = str(tmp_path / "ad1"), str(tmp_path / "ad2")
    m1 = _make_adapter(ad1, cfg, st, r=8, alpha=16, seed=1)
    m2 = _make_adapter(ad2, cfg, st, r=4, alpha=4, seed=2, targets=("q_proj", "v_proj", "down_proj"))
    prompts = _prompts(cfg, [300, 64, 200])
    cfg32 = ModelConfig(name=ARCH, **dict(MODEL_PRESETS[ARCH], dtype=torch.float32))
    want = [naive_logits(cfg32, s, p)[-1] for s, p in zip((m1, st, m2), prompts)]
    wrong = [naive_logits(cfg32, s, p)[-1] for s, p in zip((st, m1, st), prompts)]
    ep = str(tmp_path / "expect.pt")
    torch.save({"want": want, "wrong": wrong}, ep)
    run_ranks(_lora_rank, 2, ckpt, ad1, ad2, prompts, ep, timeout=300)


# ---- KV-transfer connector, caches in GPU memory (one GPU) -----------------------------------------------------
def test_kv_connector_between_gpu_engines(tmp_path):
    from tokenweave_b200 import LLM, SamplingParams, ops
    from test_kv_connector_cpu import _cfg, _prefill_tokens, _stored
    cfg, _, ckpt = _checkpoint(tmp_path, seed=31)
    store = str(tmp_path / "store")
    shared = _prompts(cfg, [300])[0]
    p1, p2 = shared + [7, 8, 9], shared + [11, 12, 13, 14, 15]
    sp = SamplingParams(temperature=0, max_tokens=4, ignore_eos=True)
    args = dict(device="cuda", skip_tokenizer_init=True, block_size=128, max_num_batched_tokens=512,
                num_gpu_blocks_override=32)
    plain = LLM(ckpt, **args)
    runner = plain.llm_engine.core.executor.worker.runner
    runner.capture_logits = True
    want = _first_rows(runner, plain.generate([p2, p1], sp)).float().cpu()
    plain.shutdown()

    producer = LLM(ckpt, kv_transfer_config=_cfg("kv_producer", store), **args)
    outs, computed = _prefill_tokens(producer, [p1], sp)
    assert computed == len(p1) + 3
    producer.shutdown()
    files = _stored(store)
    assert len(files) == len(p1) // 128                 # the two full blocks of the prompt

    consumer = LLM(ckpt, kv_transfer_config=_cfg("kv_consumer", store), **args)
    runner = consumer.llm_engine.core.executor.worker.runner
    runner.capture_logits = True
    outs2, computed2 = _prefill_tokens(consumer, [p2, p1], sp)
    torch.cuda.synchronize()
    ops.check_status()
    assert computed2 == (len(p2) - 256 + 3) + (len(p1) - 256 + 3)     # only the tails were computed
    # the tails attended to the fetched blocks: first-token logits as with a full prefill (another tile shape
    # of the same kernels, so equal up to bf16 rounding)
    torch.testing.assert_close(_first_rows(runner, outs2).float().cpu(), want, atol=3e-2, rtol=3e-2)
    assert _stored(store) == files                                      # a consumer writes nothing
    consumer.shutdown()
