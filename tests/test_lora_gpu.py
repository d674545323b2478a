"""LoRA on the GPU (bf16): adapter deltas run through the tcgen05 GEMM on gathered rows; logits must track the
fp32 model with merged weights within bf16 tolerance, for a batch that mixes two adapters and no adapter."""
import pytest
import torch

from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
from tokenweave_b200.models.loader import save_hf_checkpoint

from test_lora_cpu import _first_logits, _make_adapter
from tw_testing import hf_config_dict, make_hf_state, naive_logits

pytestmark = pytest.mark.gpu


def test_lora_mixed_batch_tracks_merged_model(tmp_path):
    from tokenweave_b200 import LLM, ops
    from tokenweave_b200.lora import LoRARequest
    arch = "tiny-llama-d128"
    cfg = ModelConfig(name=arch, **MODEL_PRESETS[arch])
    st = make_hf_state(cfg, seed=5)
    hf = hf_config_dict(cfg)
    hf["torch_dtype"] = "bfloat16"
    ckpt = str(tmp_path / "base")
    save_hf_checkpoint({k: v.to(torch.bfloat16) for k, v in st.items()}, hf, ckpt)
    st = {k: v.to(torch.bfloat16).float() for k, v in st.items()}            # what the engine actually holds
    m1 = _make_adapter(str(tmp_path / "ad1"), cfg, st, r=8, alpha=16, seed=1)
    m2 = _make_adapter(str(tmp_path / "ad2"), cfg, st, r=4, alpha=4, seed=2, targets=("q_proj", "v_proj", "down_proj"))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (300, 64, 200)]
    llm = LLM(ckpt, device="cuda", skip_tokenizer_init=True, block_size=128, max_num_batched_tokens=1024,
              num_gpu_blocks_override=64, enable_lora=True)
    lr1, lr2 = LoRARequest("one", 1, str(tmp_path / "ad1")), LoRARequest("two", 2, str(tmp_path / "ad2"))
    logits, _ = _first_logits(llm, prompts, [lr1, None, lr2])
    torch.cuda.synchronize()
    ops.check_status()
    cfg32 = ModelConfig(name=arch, **dict(MODEL_PRESETS[arch], dtype=torch.float32))
    for lg, p, state, other in zip(logits, prompts, (m1, st, m2), (st, m1, st)):
        want = naive_logits(cfg32, state, p)[-1]
        wrong = naive_logits(cfg32, other, p)[-1]
        err = (lg.float().cpu() - want).abs().max().item()
        assert err < 0.08 * max(1.0, want.abs().max().item()), err
        # and it is the adapter's model, not the other one, that the logits follow
        assert err < (lg.float().cpu() - wrong).abs().max().item()
    llm.shutdown()
