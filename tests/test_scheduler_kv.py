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


# ---- randomised runs: invariants that must hold for any arrival pattern ---------------------------
def _fuzz_once(seed, caching, spec_k, policy="fcfs"):
    import random
    from tokenweave_b200.engine.spec_decode import SpecDecodeConfig
    rng = random.Random(seed)
    block = rng.choice([4, 16])
    num_blocks = rng.randrange(12, 40)
    budget = rng.choice([16, 48, 96])
    kv = KVCacheManager(num_blocks, block, caching)
    spec = SpecDecodeConfig(num_speculative_tokens=spec_k)
    s = Scheduler(SchedulerConfig(budget, rng.randrange(2, 7), True, 512, policy), kv, spec)
    capacity = (num_blocks - 1) * block
    pending = []
    for i in range(rng.randrange(4, 14)):
        n = rng.randrange(1, min(120, capacity // 2))
        shared = [1, 2, 3, 4] * (n // 8)                 # common prefixes so that the prefix cache gets hits
        ids = (shared + [rng.randrange(5, 50) for _ in range(n)])[:n]
        pending.append(Request(str(i), ids, SamplingParams(max_tokens=rng.randrange(1, 12), temperature=0,
                                                            stop_token_ids=[49] if rng.random() < 0.3 else None)))
        pending[-1].priority = rng.randrange(0, 4) if policy == "priority" else 0
    expected_prompt = {r.request_id: list(r.prompt_token_ids) for r in pending}
    finished, steps = {}, 0
    while pending or s.has_unfinished_requests():
        steps += 1
        assert steps < 3000, "the scheduler stopped making progress"
        for _ in range(rng.randrange(0, 3)):
            if pending:
                s.add_request(pending.pop())
        if not s.has_unfinished_requests():
            continue
        out = s.schedule()
        assert out.total_num_tokens <= budget
        assert len({x.request.request_id for x in out.scheduled}) == len(out.scheduled)
        # a request preempted in this step runs no tokens in it, and what runs is in the running list
        assert not {x.request.request_id for x in out.scheduled} & set(out.preempted_req_ids)
        assert all(x.request in s.running for x in out.scheduled)
        owned = [b for r in s.running for b in r.block_ids]
        if not caching:
            assert len(owned) == len(set(owned)), "a block is owned twice"
        for x in out.scheduled:
            r = x.request
            assert x.num_new_tokens >= 1
            assert len(r.block_ids) * block >= x.num_computed_tokens + x.num_new_tokens, "not enough slots"
        toks = []
        for x in out.scheduled:
            if x.spec_token_ids:        # the model confirms a random number of drafts, then emits one more token
                keep = rng.randrange(0, len(x.spec_token_ids) + 1)
                toks.append(list(x.spec_token_ids[:keep]) + [rng.randrange(5, 50)])
            else:
                toks.append(rng.randrange(5, 50))
        touched = s.update_from_output(out, ModelRunnerOutput([x.request.request_id for x in out.scheduled], toks))
        for r in touched:
            if r.status.finished:
                finished[r.request_id] = r
        if rng.random() < 0.05 and s.running:      # a client walks away
            victim = rng.choice(s.running)
            s.abort_request(victim.request_id)
            finished[victim.request_id] = victim
    assert set(finished) == set(expected_prompt)
    for rid, r in finished.items():
        assert r.prompt_token_ids == expected_prompt[rid]
        if r.status != RequestStatus.FINISHED_ABORTED:
            assert 1 <= len(r.output_token_ids) <= r.sampling_params.max_tokens
            if r.status == RequestStatus.FINISHED_STOPPED:
                assert r.output_token_ids[-1] == 49 and 49 not in r.output_token_ids[:-1]
            else:
                assert len(r.output_token_ids) == r.sampling_params.max_tokens
        assert r.block_ids == []
    # every block is back in the pool and nothing holds a reference
    assert kv.pool.num_free == num_blocks - 1
    assert all(c == 0 for c in kv.pool.ref[1:])


@pytest.mark.parametrize("caching,spec_k", [(False, 0), (True, 0), (False, 3), (True, 2)])
def test_random_workloads_keep_the_invariants(caching, spec_k):
    for seed in range(60):
        _fuzz_once(seed * 7 + spec_k, caching, spec_k)


@pytest.mark.parametrize("caching,spec_k", [(False, 0), (True, 2)])
def test_random_workloads_under_the_priority_policy(caching, spec_k):
    for seed in range(60):
        _fuzz_once(seed * 11 + spec_k, caching, spec_k, policy="priority")


def test_priority_victim_already_scheduled_in_the_step_is_taken_out():
    """A less urgent request that got its tokens earlier in the step loses them (and its blocks) when a more
    urgent one behind it in the running list cannot grow: it must not stay among the step's scheduled requests."""
    kv = KVCacheManager(num_blocks=7, block_size=16, enable_caching=False)       # 6 usable blocks
    s = Scheduler(SchedulerConfig(64, 8, True, 1024, "priority"), kv)
    a, b = req(0, 34, max_tokens=40), req(1, 47, max_tokens=40)
    a.priority, b.priority = 5, 0
    s.add_request(a)
    run_step(s)
    s.add_request(b)
    seen = False
    for _ in range(6):
        out = s.schedule()
        ids = [x.request.request_id for x in out.scheduled]
        assert not set(ids) & set(out.preempted_req_ids)
        assert out.total_num_tokens == sum(x.num_new_tokens for x in out.scheduled) <= 64
        owned = [blk for r in s.running for blk in r.block_ids]
        assert len(owned) == len(set(owned))
        seen = seen or out.preempted_req_ids == ["0"]
        s.update_from_output(out, ModelRunnerOutput(ids, [7] * len(ids)))
    assert seen, "the case never preempted the less urgent request"
    assert a.status == RequestStatus.PREEMPTED or a in s.running


def test_priority_policy_orders_admission_and_preemption():
    kv = KVCacheManager(num_blocks=12, block_size=16, enable_caching=False)
    s = Scheduler(SchedulerConfig(64, 8, True, 1024, "priority"), kv)
    for i, prio in enumerate([5, 1, 3, 1]):
        r = req(i, 40, max_tokens=50)
        r.priority = prio
        s.add_request(r)
    assert [r.request_id for r in s.waiting] == ["1", "3", "2", "0"]        # by priority, arrival among equals
    out, _ = run_step(s)
    assert [x.request.request_id for x in out.scheduled] == ["1", "3"]      # 40 + 24 tokens of the 64-token budget
    for _ in range(3):
        run_step(s)
    assert {r.request_id for r in s.running} >= {"1", "3", "2"}
    # the pool (11 usable blocks) runs dry while three requests decode: the least urgent of them is the victim
    victims = []
    for _ in range(40):
        out, _ = run_step(s)
        victims += out.preempted_req_ids
        if victims:
            break
    assert victims and victims[0] == "2" and "1" not in victims and "3" not in victims
    with pytest.raises(ValueError):
        Scheduler(SchedulerConfig(64, 8, True, 1024, "lottery"), kv).add_request(req(9, 4))


def test_long_prefill_threshold_lets_short_requests_in():
    """With a cap on the new tokens of one request per step a long prompt shares the budget from the first step."""
    kv = KVCacheManager(64, 16, False)
    s = Scheduler(SchedulerConfig(64, 8, True, 1024, "fcfs", 24), kv)
    s.add_request(req(0, 100))
    s.add_request(req(1, 30))
    out, _ = run_step(s)
    assert [(x.request.request_id, x.num_new_tokens) for x in out.scheduled] == [("0", 24), ("1", 24)]
    out, touched = run_step(s)
    # both continue under the cap; request 1 finishes its prompt with its last six tokens and emits a token
    assert [(x.request.request_id, x.num_new_tokens) for x in out.scheduled] == [("0", 24), ("1", 6)]
    assert [r.request_id for r in touched] == ["1"]
    steps = 2
    while s.has_unfinished_requests() and steps < 40:
        run_step(s)
        steps += 1
    assert not s.has_unfinished_requests() and kv.pool.num_free == 63      # everything finished, blocks returned
    # without chunked prefill the cap is ignored (a prompt is scheduled whole or not at all)
    kv2 = KVCacheManager(64, 16, False)
    s2 = Scheduler(SchedulerConfig(128, 8, False, 1024, "fcfs", 24), kv2)
    s2.add_request(req(0, 100))
    out, _ = run_step(s2)
    assert [(x.request.request_id, x.num_new_tokens) for x in out.scheduled] == [("0", 100)]
