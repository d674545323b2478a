"""StoreGroup: a control-plane process group on a TCP store, independent of torch.distributed's global state."""
import pytest

from tw_testing import free_port, run_ranks


def _rank(rank, world, port):
    import torch.distributed as dist
    from tokenweave_b200.parallel.store_group import StoreGroup
    g = StoreGroup.create("127.0.0.1", port, rank, world, timeout_s=30)
    assert not dist.is_initialized()                      # no global process group is created
    # two groups on one store do not collide when their keys are prefixed
    g2 = StoreGroup(dist.PrefixStore("second", g.store), rank, world, timeout_s=30)
    for round_ in range(3):
        got = g.all_gather_obj({"rank": rank, "round": round_})
        assert got == [{"rank": r, "round": round_} for r in range(world)]
        assert g2.broadcast_obj(("hello", round_) if rank == 1 else None, src=1) == ("hello", round_)
        g.barrier()
    # a ring of point-to-point messages, two in flight per pair
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    g.send_obj([rank, "a"], nxt)
    g.send_obj([rank, "b"], nxt)
    assert g.recv_obj(prv) == [prv, "a"] and g.recv_obj(prv) == [prv, "b"]
    g.barrier()
    # a rank that never arrives: the others get an error, not a hang
    if rank != 2:
        with pytest.raises(TimeoutError):
            g.barrier(timeout_s=0.3)
    with pytest.raises(TimeoutError):
        g2.recv_obj(src=(rank + 1) % world, timeout_s=0.2)
    g2.barrier()                                           # keep the store's host alive until everyone is done


def test_store_group_collectives_and_timeouts():
    run_ranks(_rank, 3, free_port())
