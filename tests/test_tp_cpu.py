"""Tensor parallelism and the executors on CPU (gloo, world size 2): every schedule must reproduce the
single-process result from the same checkpoint; worker failures must surface as EngineDeadError."""
import os

import pytest
import torch

from tokenweave_b200 import LLM, SamplingParams
from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
from tokenweave_b200.models.loader import save_hf_checkpoint

from tw_testing import hf_config_dict, make_hf_state, run_ranks


def _ckpt(tmp_path, arch="tiny-llama", **over):
    preset = dict(MODEL_PRESETS[arch])
    preset.update(hidden_size=128, head_dim=32, intermediate_size=192, vocab_size=320, max_model_len=1024)
    preset.update(over)
    cfg = ModelConfig(name=arch, **preset)
    st = make_hf_state(cfg, seed=3)
    save_hf_checkpoint(st, hf_config_dict(cfg), str(tmp_path))
    return cfg


def _prompts(vocab, lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def _generate(path, prompts, **kw):
    args = dict(dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=512)
    args.update(kw)
    llm = LLM(path, **args)
    runner = None
    try:
        runner = llm.llm_engine.core.executor.worker.runner
        runner.capture_logits = True
    except AttributeError:
        pass
    outs = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=6))
    toks = [o.outputs[0].token_ids for o in outs]
    logits = torch.cat([l for _, l in runner.captured_logits]) if runner is not None else None
    llm.shutdown()
    return toks, logits


def _spmd_rank(rank, world, path, prompts, mode, expect_toks, expect_logits_path, emb_parallel):
    if emb_parallel:
        os.environ["TW_EMBEDDING_PARALLEL"] = "1"
    toks, logits = _generate(path, prompts, tensor_parallel_size=world, distributed_executor_backend="external_launcher",
                             tokenweave_mode=mode, tokenweave_threshold=128)
    assert toks == expect_toks, f"rank {rank} mode {mode}: {toks} != {expect_toks}"
    torch.testing.assert_close(logits, torch.load(expect_logits_path), atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("arch,mode,emb_parallel", [
    ("tiny-llama", "overlap", False), ("tiny-llama", "fuse_only", True), ("tiny-llama", "baseline_nccl", False),
    ("tiny-qwen2", "overlap", True), ("tiny-mixtral", "overlap", False), ("tiny-llama", "fused_gemm", False),
    ("tiny-mixtral", "fused_gemm", False)])
def test_spmd_tp2_matches_single_process(tmp_path, arch, mode, emb_parallel):
    cfg = _ckpt(tmp_path, arch)
    prompts = _prompts(cfg.vocab_size, [150, 40, 90, 9])      # 289 tokens: overlap schedule with a straddling request
    toks, logits = _generate(str(tmp_path), prompts)
    lp = str(tmp_path / "expect_logits.pt")
    torch.save(logits, lp)
    run_ranks(_spmd_rank, 2, str(tmp_path), prompts, mode, toks, lp, emb_parallel)


def test_kv_head_replication_tp4(tmp_path):
    cfg = _ckpt(tmp_path, "tiny-llama", num_q_heads=4, num_kv_heads=2)
    prompts = _prompts(cfg.vocab_size, [70, 20])
    toks, logits = _generate(str(tmp_path), prompts)
    lp = str(tmp_path / "expect_logits.pt")
    torch.save(logits, lp)
    run_ranks(_spmd_rank, 4, str(tmp_path), prompts, "fuse_only", toks, lp, False)


def test_multiproc_executor_matches_and_shuts_down(tmp_path):
    cfg = _ckpt(tmp_path)
    prompts = _prompts(cfg.vocab_size, [150, 40, 90])
    toks, _ = _generate(str(tmp_path), prompts)
    got, _ = _generate(str(tmp_path), prompts, tensor_parallel_size=2, distributed_executor_backend="mp",
                       tokenweave_threshold=128)
    assert got == toks


@pytest.mark.parametrize("var", ["TW_TEST_FAIL_AT_STEP", "TW_TEST_EXIT_AT_STEP"])
def test_worker_failure_surfaces_as_engine_dead(tmp_path, monkeypatch, var):
    """A worker that raises in execute_model, or exits between steps, ends generate() with
    EngineDeadError instead of a hang (host-side fault injection; no device is involved)."""
    from tokenweave_b200.engine.core import EngineDeadError
    cfg = _ckpt(tmp_path)
    monkeypatch.setenv(var, "3")
    monkeypatch.setenv("TW_TEST_FAULT_RANK", "1")
    monkeypatch.setenv("TW_EXECUTE_MODEL_TIMEOUT_S", "20")
    llm = LLM(str(tmp_path), dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16,
              max_num_batched_tokens=256, tensor_parallel_size=2, distributed_executor_backend="mp")
    with pytest.raises(EngineDeadError):
        llm.generate(_prompts(cfg.vocab_size, [30, 30]), SamplingParams(temperature=0, max_tokens=8))
    with pytest.raises(EngineDeadError):
        llm.generate(_prompts(cfg.vocab_size, [5]), SamplingParams(max_tokens=1))
    llm.shutdown()


def test_message_queue_large_payload_and_timeout():
    from tokenweave_b200.parallel.shm_broadcast import MessageQueue
    w = MessageQueue.create(n_readers=2, chunk_bytes=1024, num_chunks=4)
    r0, r1 = MessageQueue.attach(w.handle(), 0), MessageQueue.attach(w.handle(), 1)
    big = {"x": list(range(3000))}
    import threading
    got = []
    ts = [threading.Thread(target=lambda q=q: got.append(q.dequeue(timeout=10))) for q in (r0, r1)]
    for t in ts:
        t.start()
    w.enqueue(big, timeout=10)
    for t in ts:
        t.join()
    assert got == [big, big]
    with pytest.raises(TimeoutError):
        r0.dequeue(timeout=0.05)
    for q in (r0, r1, w):
        q.close()


def test_engines_built_one_after_another_under_torchrun(tmp_path):
    """Several engines in one torchrun job (what the benchmark scripts do, one per schedule): every
    re-initialisation of the process group must use fresh rendezvous keys in the launcher's store."""
    import subprocess
    import sys
    from tw_testing import free_port
    script = tmp_path / "reinit.py"
    script.write_text(
        "import os\n"
        "from tokenweave_b200 import LLM, SamplingParams\n"
        "for i in range(3):\n"
        "    llm = LLM('tiny-llama', dtype='float32', device='cpu', tensor_parallel_size=2, skip_tokenizer_init=True,\n"
        "              distributed_executor_backend='external_launcher', block_size=16, max_num_batched_tokens=128)\n"
        "    out = llm.generate(prompt_token_ids=[[1, 2, 3, 4, 5]], sampling_params=SamplingParams(temperature=0, max_tokens=3))\n"
        "    if os.environ['RANK'] == '0':\n"
        "        print('RESULT', i, out[0].outputs[0].token_ids, flush=True)\n"
        "    llm.shutdown()\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(free_port()), str(script)],
                         env=env, capture_output=True, text=True, timeout=280)
    assert res.returncode == 0, res.stderr[-3000:]
    lines = [ln.split(" ", 2)[2] for ln in res.stdout.splitlines() if ln.startswith("RESULT")]
    assert len(lines) == 3 and len(set(lines)) == 1


def _ep_rank(rank, world, path, prompts, expect_toks, expect_logits_path):
    toks, logits = _generate(path, prompts, tensor_parallel_size=world, distributed_executor_backend="external_launcher",
                             tokenweave_mode="overlap", tokenweave_threshold=128, enable_expert_parallel=True)
    assert toks == expect_toks, f"rank {rank}: {toks} != {expect_toks}"
    torch.testing.assert_close(logits, torch.load(expect_logits_path), atol=2e-4, rtol=2e-4)


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_mixtral_matches_single_process(tmp_path, world):
    """enable_expert_parallel: every rank holds whole experts (8 / world each) and the partial sums meet in
    the same fused reduce-scatter as tensor-sharded experts; results equal the single-process model."""
    cfg = _ckpt(tmp_path, "tiny-mixtral")
    prompts = _prompts(cfg.vocab_size, [150, 40, 90, 9])
    toks, logits = _generate(str(tmp_path), prompts)
    lp = str(tmp_path / "expect_logits.pt")
    torch.save(logits, lp)
    run_ranks(_ep_rank, world, str(tmp_path), prompts, toks, lp)


def _spec_rank(rank, world, path, prompts, expect_toks):
    toks, _ = _generate(path, prompts, tensor_parallel_size=world, distributed_executor_backend="external_launcher",
                        tokenweave_mode="overlap", tokenweave_threshold=128, speculative_config=4)
    assert toks == expect_toks, f"rank {rank}: {toks} != {expect_toks}"


def test_speculative_decoding_under_tp2_matches_plain_single_process(tmp_path):
    """Every SPMD rank drafts and verifies the same tokens (the proposer is a pure function of the history)."""
    cfg = _ckpt(tmp_path, "tiny-llama")
    g = torch.Generator().manual_seed(4)
    base = torch.randint(0, cfg.vocab_size, (20,), generator=g).tolist()
    prompts = [base * 6, base[:9] * 5, torch.randint(0, cfg.vocab_size, (150,), generator=g).tolist()]
    toks, _ = _generate(str(tmp_path), prompts)
    run_ranks(_spec_rank, 2, str(tmp_path), prompts, toks)
