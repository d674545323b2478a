"""KV-transfer connector on CPU: a producer engine publishes the blocks of a prompt to shared storage; a consumer
engine with an empty cache picks them up, computes only what is missing and generates the same tokens."""
import os

import pytest
import torch

from tokenweave_b200 import LLM, SamplingParams
from tokenweave_b200.config import MODEL_PRESETS, ModelConfig
from tokenweave_b200.engine.kv_connector import KVTransferConfig
from tokenweave_b200.models.loader import save_hf_checkpoint

from tw_testing import hf_config_dict, make_hf_state, naive_logits


def _cfg(role, path):
    return {"kv_connector": "SharedStorageConnector", "kv_role": role,
            "kv_connector_extra_config": {"shared_storage_path": path}}


def _prefill_tokens(llm, prompts, sp):
    """Run and count the tokens the engine actually computed (scheduled) for these requests."""
    total = 0
    orig = llm.llm_engine.core.scheduler.schedule

    def counting():
        nonlocal total
        out = orig()
        total += out.total_num_tokens
        return out
    llm.llm_engine.core.scheduler.schedule = counting
    outs = llm.generate(prompts, sp)
    llm.llm_engine.core.scheduler.schedule = orig
    return outs, total


def _stored(store):
    return sorted(f for _, _, names in os.walk(store) for f in names)


def test_consumer_reuses_the_producers_blocks(tmp_path):
    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    st = make_hf_state(cfg, seed=31)
    ckpt, store = str(tmp_path / "ckpt"), str(tmp_path / "store")
    save_hf_checkpoint(st, hf_config_dict(cfg), ckpt)
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, cfg.vocab_size, (100,), generator=g).tolist()
    p1, p2 = shared + [7, 8, 9], shared + [11, 12, 13, 14, 15]
    sp = SamplingParams(temperature=0, max_tokens=4, ignore_eos=True)
    args = dict(dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=64)

    producer = LLM(ckpt, kv_transfer_config=_cfg("kv_producer", store), **args)
    outs, computed = _prefill_tokens(producer, [p1], sp)
    assert computed == len(p1) + 3                       # prompt + the decode steps
    producer.shutdown()
    files = _stored(store)
    assert len(os.listdir(store)) == 1                   # one sub-directory: the fingerprint of this KV layout
    assert len(files) == len(p1) // 16 and all(f.endswith(".r0of1.pt") for f in files)

    consumer = LLM(ckpt, kv_transfer_config=_cfg("kv_consumer", store), **args)
    outs2, computed2 = _prefill_tokens(consumer, [p2, p1], sp)
    # six blocks (96 tokens) of each prompt came from the store; only the tails were computed
    assert computed2 == (len(p2) - 96 + 3) + (len(p1) - 96 + 3)
    for out, p in zip(outs2, (p2, p1)):
        seq = list(p)
        for _ in range(4):
            seq.append(int(naive_logits(cfg, st, seq)[-1].argmax()))
        assert out.outputs[0].token_ids == seq[len(p):]
    assert outs2[1].outputs[0].token_ids == outs[0].outputs[0].token_ids
    assert _stored(store) == files                       # a consumer writes nothing
    consumer.shutdown()


def test_bad_connector_configs_are_refused(tmp_path):
    with pytest.raises(ValueError):
        KVTransferConfig.from_user({"kv_connector": "Other", "kv_connector_extra_config": {"shared_storage_path": "x"}})
    with pytest.raises(ValueError):
        KVTransferConfig.from_user({"kv_role": "kv_reader", "kv_connector_extra_config": {"shared_storage_path": "x"}})
    with pytest.raises(ValueError):
        KVTransferConfig.from_user({"kv_role": "kv_both"})


def _tp_rank(rank, world, ckpt, store, p1, p2, expect):
    import torch.distributed as dist
    sp = SamplingParams(temperature=0, max_tokens=4, ignore_eos=True)
    llm = LLM(ckpt, kv_transfer_config=_cfg("kv_both", store), dtype="float32", device="cpu", skip_tokenizer_init=True,
              block_size=16, max_num_batched_tokens=64, tensor_parallel_size=world,
              distributed_executor_backend="external_launcher")
    llm.generate([p1], sp)
    assert llm.reset_prefix_cache()          # the local cache forgets everything: what follows comes from the store
    dist.barrier()                           # both ranks' files are there before either looks them up
    outs, computed = _prefill_tokens(llm, [p2], sp)
    assert computed == len(p2) - 96 + 3, computed
    assert outs[0].outputs[0].token_ids == expect
    llm.shutdown()


def test_connector_under_tp2(tmp_path):
    from tw_testing import run_ranks
    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    st = make_hf_state(cfg, seed=32)
    ckpt, store = str(tmp_path / "ckpt"), str(tmp_path / "store")
    save_hf_checkpoint(st, hf_config_dict(cfg), ckpt)
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, cfg.vocab_size, (100,), generator=g).tolist()
    p1, p2 = shared + [3, 4], shared + [5, 6, 7]
    seq = list(p2)
    for _ in range(4):
        seq.append(int(naive_logits(cfg, st, seq)[-1].argmax()))
    run_ranks(_tp_rank, 2, ckpt, store, p1, p2, seq[len(p2):])
    assert len(_stored(store)) == 2 * 6              # six blocks, one file per rank


def test_blocks_travel_through_a_tcp_store(tmp_path):
    """TcpStoreConnector: the producer engine hosts a key-value store, the consumer connects to it over a socket,
    finds the producer's blocks and computes only the tail of its prompts."""
    from tw_testing import free_port
    from tokenweave_b200.engine.kv_connector import decode_block, encode_block
    k = torch.randn(2, 16, 2, 8).to(torch.bfloat16)
    k2, v2 = decode_block(encode_block(k, k + 1))
    assert torch.equal(k2, k) and torch.equal(v2, k + 1) and k2.dtype == torch.bfloat16
    with pytest.raises(ValueError):
        decode_block(encode_block(k, k)[:-4])

    cfg = ModelConfig(name="tiny-llama", **MODEL_PRESETS["tiny-llama"])
    st = make_hf_state(cfg, seed=33)
    ckpt = str(tmp_path / "ckpt")
    save_hf_checkpoint(st, hf_config_dict(cfg), ckpt)
    port = free_port()

    def tcp(role, host, master):
        return {"kv_connector": "TcpStoreConnector", "kv_role": role,
                "kv_connector_extra_config": {"host": host, "port": port, "is_master": master, "timeout_s": 20}}

    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, cfg.vocab_size, (100,), generator=g).tolist()
    p1, p2 = shared + [7, 8, 9], shared + [11, 12, 13, 14, 15]
    sp = SamplingParams(temperature=0, max_tokens=4, ignore_eos=True)
    args = dict(dtype="float32", device="cpu", skip_tokenizer_init=True, block_size=16, max_num_batched_tokens=64)
    producer = LLM(ckpt, kv_transfer_config=tcp("kv_producer", "127.0.0.1", True), **args)
    try:
        outs, computed = _prefill_tokens(producer, [p1], sp)
        assert computed == len(p1) + 3
        # "localhost" instead of "127.0.0.1": the consumer does not find the store object of this process and
        # goes through the socket, as an engine on another machine would
        consumer = LLM(ckpt, kv_transfer_config=tcp("kv_consumer", "localhost", False), **args)
        try:
            outs2, computed2 = _prefill_tokens(consumer, [p2, p1], sp)
            assert computed2 == (len(p2) - 96 + 3) + (len(p1) - 96 + 3)        # six blocks of each prompt came over
            for out, p in zip(outs2, (p2, p1)):
                seq = list(p)
                for _ in range(4):
                    seq.append(int(naive_logits(cfg, st, seq)[-1].argmax()))
                assert out.outputs[0].token_ids == seq[len(p):]
        finally:
            consumer.shutdown()
    finally:
        producer.shutdown()
    with pytest.raises(ValueError):
        KVTransferConfig.from_user({"kv_connector": "TcpStoreConnector", "kv_role": "kv_both"})          # no port
    with pytest.raises(ValueError):
        KVTransferConfig.from_user({"kv_connector": "Carrier pigeon", "kv_role": "kv_both"})
