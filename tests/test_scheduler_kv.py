"""Scheduler and KV-cache manager (CPU only, no model): token budget, chunked prefill, preemption by
recompute, prefix-cache hits, block accounting."""
import pytest

from tokenweave_b200.config import SchedulerConfig
from tokenweave_b200.engine.kv_cache import BlockPool, KVCacheManager, block_hashes
from tokenweave_b200.engine.request import Request, RequestStatus
from tokenweave_b200.engine.scheduler import ModelRunnerOutput, Scheduler
from tokenweave_b200.sampling_params import SamplingParams


def make(num_blocks=64, block=16, budget=64, max_seqs=8, caching=False, chunked=True, max_len=1024):
    kv = KVCacheManager(num_blocks, block, caching)
    return Scheduler(SchedulerConfig(budget, max_seqs, chunked, max_len), kv), kv


def req(i, n_prompt, max_tokens=4, base=0):
    return Request(str(i), [base + j for j in range(n_prompt)], SamplingParams(max_tokens=max_tokens, temperature=0))


def run_step(s, token=7):
    out = s.schedule()
    res = ModelRunnerOutput([x.request.request_id for x in out.scheduled], [token] * len(out.scheduled))
    return out, s.update_from_output(out, res)


def test_budget_and_chunked_prefill():
    s, kv = make(budget=64)
    s.add_request(req(0, 100))
    s.add_request(req(1, 30))
    out, touched = run_step(s)
    assert [(x.request.request_id, x.num_new_tokens) for x in out.scheduled] == [("0", 64)]
    assert touched == []                      # still prefilling: the sampled token is discarded
    out, touched = run_step(s)
    assert [(x.request.request_id, x.num_new_tokens) for x in out.scheduled] == [("0", 36), ("1", 28)]
    assert [r.request_id for r in touched] == ["0"]
    out, touched = run_step(s)
    # request 0 decodes one token, request 1 finishes its prompt
    assert [(x.request.request_id, x.num_new_tokens) for x in out.scheduled] == [("0", 1), ("1", 2)]
    assert sorted(r.request_id for r in touched) == ["0", "1"]


def test_finish_by_length_and_blocks_freed():
    s, kv = make()
    s.add_request(req(0, 20, max_tokens=3))
    free0 = kv.pool.num_free
    for _ in range(3):
        run_step(s)
    assert not s.has_unfinished_requests()
    assert kv.pool.num_free == free0
    assert s.schedule().finished_req_ids == ["0"]


def test_eos_and_stop_token():
    s, kv = make()
    r = req(0, 5, max_tokens=10)
    r.eos_token_id = 7
    s.add_request(r)
    run_step(s, token=7)
    assert r.status == RequestStatus.FINISHED_STOPPED and r.finish_reason == "stop"
    r2 = Request("1", [1, 2, 3], SamplingParams(max_tokens=10, stop_token_ids=[9]))
    s.add_request(r2)
    run_step(s, token=9)
    assert r2.status == RequestStatus.FINISHED_STOPPED and r2.stop_reason == 9


def test_preemption_by_recompute():
    s, kv = make(num_blocks=6, block=16, budget=256)     # 5 usable blocks = 80 tokens
    a, b = req(0, 40, max_tokens=50), req(1, 30, max_tokens=50, base=100)
    s.add_request(a)
    s.add_request(b)
    run_step(s)                                        # both prefill: 3 + 2 blocks
    assert len(s.running) == 2
    preempted_seen = False
    for _ in range(12):
        out, _ = run_step(s)
        preempted_seen |= bool(out.preempted_req_ids)
        if preempted_seen:
            break
    assert preempted_seen
    assert b.status == RequestStatus.PREEMPTED and b.num_computed_tokens == 0 and b.block_ids == []
    assert s.waiting[0] is b


def test_prefix_cache_hit():
    s, kv = make(num_blocks=64, block=16, budget=256, caching=True)
    s.add_request(req(0, 50, max_tokens=1))
    run_step(s)
    assert not s.has_unfinished_requests()
    r = req(1, 50, max_tokens=1)
    s.add_request(r)
    out = s.schedule()
    assert out.scheduled[0].num_computed_tokens == 48 and out.scheduled[0].num_new_tokens == 2


def test_block_pool_refcount_and_hash_chain():
    pool = BlockPool(8, enable_caching=True)
    blocks = pool.allocate(3)
    assert 0 not in blocks and pool.num_free == 4
    pool.cache_block(blocks[0], b"h0")
    pool.release(blocks)
    assert pool.num_free == 7 and pool.lookup(b"h0") == blocks[0]
    pool.touch(blocks[0])
    assert pool.num_free == 6
    h1, h2 = block_hashes(list(range(32)), 16), block_hashes(list(range(16)) + [99] * 16, 16)
    assert h1[0] == h2[0] and h1[1] != h2[1]


def test_prompt_too_long_rejected():
    s, _ = make(max_len=32)
    with pytest.raises(ValueError):
        s.add_request(req(0, 40))
