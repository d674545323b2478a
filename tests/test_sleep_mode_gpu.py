"""Sleep mode on the VMM allocator: physical memory is released while tensors keep their addresses;
tagged contents come back after wake-up; an engine generates the same tokens before and after."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pool_sleep_and_wake_keep_addresses_and_tagged_contents():
    from tokenweave_b200.utils.sleep_allocator import TAG_KV_CACHE, TAG_WEIGHTS, SleepAllocator
    alloc = SleepAllocator.get()
    with alloc.use_pool(TAG_WEIGHTS):
        w = torch.arange(64 << 20, dtype=torch.int32, device="cuda")          # 256 MiB, kept
    with alloc.use_pool(TAG_KV_CACHE):
        kv = torch.ones(128 << 20, dtype=torch.bfloat16, device="cuda")       # 256 MiB, discarded
    outside = torch.full((1024,), 7, device="cuda")
    ptrs = (w.data_ptr(), kv.data_ptr())
    assert alloc.mapped_bytes() >= 512 << 20
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    alloc.sleep(offload_tags=(TAG_WEIGHTS,))
    free1 = torch.cuda.mem_get_info()[0]
    assert free1 - free0 >= 500 << 20, "sleep must hand the physical memory back to the driver"
    assert alloc.mapped_bytes() == 0 and alloc.host_bytes() >= 256 << 20
    assert int(outside.sum()) == 7 * 1024               # ordinary allocations are untouched and usable
    alloc.wake_up()
    assert (w.data_ptr(), kv.data_ptr()) == ptrs
    assert alloc.mapped_bytes() == alloc.reserved_bytes() and alloc.host_bytes() == 0
    assert torch.equal(w[:1000].cpu(), torch.arange(1000, dtype=torch.int32))
    assert int(w[-1]) == (64 << 20) - 1
    kv.fill_(2)                                           # discarded contents: memory is writable again
    assert float(kv[12345]) == 2.0
    del w, kv
    torch.cuda.synchronize()


@pytest.mark.parametrize("level", [1, 2])
def test_engine_sleep_wake_round_trip(level):
    from tokenweave_b200 import LLM, SamplingParams, ops
    llm = LLM("tiny-llama-d128", device="cuda", skip_tokenizer_init=True, max_num_batched_tokens=1024, block_size=128,
              num_gpu_blocks_override=64, seed=0, enable_sleep_mode=True, enable_prefix_caching=True)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (300, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=8)
    before = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    llm.sleep(level=level)
    assert torch.cuda.mem_get_info()[0] > free0
    llm.wake_up()
    after = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]     # same seed: level 2 re-draws the same weights
    ops.check_status()
    assert after == before
    llm.shutdown()
