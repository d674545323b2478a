"""The ctypes NCCL binding: library discovery and version anywhere; collectives on two GPUs against torch's."""
import pytest
import torch

from tokenweave_b200.parallel.pynccl import NCCLLibrary, find_library

from tw_testing import run_ranks


def test_library_loads_and_reports_its_version():
    lib = NCCLLibrary()
    major = int(lib.version().split(".")[0])
    assert major >= 2 and lib.path == find_library()
    with pytest.raises(RuntimeError, match="NCCL error"):
        lib.check(5)


def _rank(rank, world):
    import torch.distributed as dist
    from tokenweave_b200.parallel import state as pstate
    from tokenweave_b200.parallel.pynccl import NcclCommunicator
    tp = pstate.init_distributed(rank, world, rank, "cuda")
    comm = NcclCommunicator(rank, world, tp.device, pstate.broadcast_object)
    x = torch.full((1 << 16,), float(rank + 1), device=tp.device, dtype=torch.bfloat16)
    comm.all_reduce(x)
    assert torch.all(x == sum(range(1, world + 1)))
    part = torch.full((1024,), float(rank), device=tp.device)
    gathered = torch.empty(world * 1024, device=tp.device)
    comm.all_gather(gathered, part)
    assert torch.equal(gathered.view(world, 1024)[:, 0].cpu(), torch.arange(world, dtype=torch.float32))
    out = torch.empty(1024, device=tp.device)
    comm.reduce_scatter(out, gathered.clone())
    assert torch.all(out == rank * world)
    if rank == 0:
        comm.send(part + 7, 1)
    elif rank == 1:
        got = torch.empty_like(part)
        comm.recv(got, 0)
        assert torch.all(got == 7)
    # captured in a CUDA graph and replayed
    g = torch.cuda.CUDAGraph()
    y = torch.ones(4096, device=tp.device)
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        comm.all_reduce(y)
    y.fill_(1.0)
    g.replay()
    torch.cuda.synchronize()
    assert torch.all(y == world)
    comm.destroy()
    dist.barrier()
    pstate.destroy_distributed()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_collectives_against_known_sums(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_ranks(_rank, world)
