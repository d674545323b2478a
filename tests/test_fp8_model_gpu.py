"""quantization="fp8" / "int8" on the GPU: the decoder linears run the 8-bit tcgen05 GEMMs on per-token quantised
activations; the logits must track the bf16 model's."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _first_logits(quant):
    from tokenweave_b200 import LLM, SamplingParams, ops
    llm = LLM("tiny-llama-d128", device="cuda", skip_tokenizer_init=True, max_num_batched_tokens=1024, block_size=128,
              num_gpu_blocks_override=64, seed=0, quantization=quant)
    runner = llm.llm_engine.core.executor.worker.runner
    runner.capture_logits = True
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (300, 64, 17)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=4))
    torch.cuda.synchronize()
    ops.check_status()
    logits = torch.cat([lg.float().cpu() for _, lg in runner.captured_logits])
    weights = {m.weight.dtype for m in runner.model.modules() if hasattr(m, "weight_scale")}
    toks = [o.outputs[0].token_ids for o in outs]
    llm.shutdown()
    return logits, weights, toks


@pytest.mark.parametrize("quant,dtype", [("fp8", torch.float8_e4m3fn), ("int8", torch.int8)])
def test_fp8_model_tracks_bf16_model(quant, dtype):
    ref, w_ref, _ = _first_logits(None)
    q, w_q, toks = _first_logits(quant)
    assert w_ref == {torch.bfloat16} and w_q == {dtype}
    cos = torch.nn.functional.cosine_similarity(ref, q, dim=-1)
    assert cos.min() > 0.97, cos
    assert all(len(t) == 4 for t in toks)
