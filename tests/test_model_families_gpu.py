"""Model families on one GPU in bf16 against the naive fp32 model of the same (bf16-rounded) weights."""
import pytest
import torch

from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
from tokenweave_b200.models.loader import save_hf_checkpoint

from tw_testing import hf_config_dict, make_hf_state, naive_logits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("arch", ["tiny-qwen3", "tiny-qwen2", "tiny-llama-d128"])
def test_first_token_logits_track_the_naive_model(tmp_path, arch):
    from tokenweave_b200 import LLM, SamplingParams, ops
    cfg = ModelConfig(name=arch, **MODEL_PRESETS[arch])
    st = make_hf_state(cfg, seed=9, dtype=torch.bfloat16)
    hf = hf_config_dict(cfg)
    hf["torch_dtype"] = "bfloat16"
    save_hf_checkpoint(st, hf, str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (260, 31, 129)]
    llm = LLM(str(tmp_path), device="cuda", skip_tokenizer_init=True, block_size=128, max_num_batched_tokens=1024,
              num_gpu_blocks_override=64)
    assert llm.llm_engine.config.model.architecture == cfg.architecture
    r = llm.llm_engine.core.executor.worker.runner
    r.capture_logits = True
    llm.generate(prompts, SamplingParams(temperature=0, max_tokens=2))
    torch.cuda.synchronize()
    ops.check_status()
    first = {}
    for reqs, logits in r.captured_logits:
        for rid, row in zip(reqs, logits):
            first.setdefault(rid, row)
    cfg32 = ModelConfig(name=arch, **dict(MODEL_PRESETS[arch], dtype=torch.float32))
    st32 = {k: v.float() for k, v in st.items()}
    for i, p in enumerate(prompts):
        want = naive_logits(cfg32, st32, p)[-1]
        err = (first[str(i)].float().cpu() - want).abs().max().item()
        assert err < 0.08 * max(1.0, want.abs().max().item()), (arch, i, err)
    llm.shutdown()
