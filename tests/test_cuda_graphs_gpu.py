"""CUDA-graph replay of repeated step shapes must reproduce the eager results."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(graphs: bool):
    from tokenweave_b200 import LLM, SamplingParams, ops
    llm = LLM("tiny-llama-d128", device="cuda", skip_tokenizer_init=True, max_num_batched_tokens=1024, block_size=128,
              num_gpu_blocks_override=64, seed=0, tokenweave_cuda_graphs=graphs)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (200, 64, 17, 300)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=24))
    outs2 = llm.generate(prompts[:1], SamplingParams(temperature=0.0, max_tokens=8))
    torch.cuda.synchronize()
    ops.check_status()
    runner = llm.llm_engine.core.executor.worker.runner
    replays = runner.graph_replays
    res = [o.outputs[0].token_ids for o in outs] + [outs2[0].outputs[0].token_ids]
    llm.shutdown()
    return res, replays


def test_graph_replay_matches_eager():
    eager, r0 = _run(False)
    graphed, r1 = _run(True)
    assert r0 == 0 and r1 >= 10, f"expected decode steps to be replayed from graphs, got {r1}"
    assert graphed == eager
