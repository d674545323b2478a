"""In-kernel collectives on 2+ GPUs (one process per GPU, NCCL for the plumbing): the fused
reduce-scatter + residual-add + RMSNorm + all-gather against NCCL all-reduce followed by the reference
add+RMSNorm, the stand-alone collectives against NCCL, over both transports (NVLS multimem and peer
loads/stores), and the bounded wait that reports instead of hanging."""
import os

import pytest
import torch

from tw_testing import run_ranks

pytestmark = pytest.mark.gpu


def _need_gpus(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _comm_worker(rank, world, transport):
    import torch.distributed as dist
    from tokenweave_b200 import ops
    from tokenweave_b200.ops import reference as ref
    from tokenweave_b200.parallel import state as pstate
    from tokenweave_b200.parallel.comm import TPCommunicator
    from tokenweave_b200.parallel.symm_mem import create_symmetric_buffer

    if transport == "p2p":
        os.environ["TW_DISABLE_NVLS"] = "1"
    if transport.startswith("native"):
        os.environ["TW_SYMM_PROVIDER"] = "native"
        if transport == "native-p2p":
            os.environ["TW_DISABLE_NVLS"] = "1"
    tp = pstate.init_distributed(rank, world, rank, "cuda")
    errors = []
    try:
        H, rows = 8192, 4096 + 512
        buf = create_symmetric_buffer(rows, H, torch.bfloat16, tp)
        comm = TPCommunicator(buf, tp, wait_budget_ms=3000, transport="auto")
        assert comm.in_kernel
        if transport in ("multimem", "native") and not comm.use_mc:
            errors.append("no multicast mapping on this machine")
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        w = (1 + 0.1 * torch.randn(H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7))).to(torch.bfloat16)
        for T, ctas, rows_in_flight, mode in [(64, 2, 1, 0), (256, 8, 0, 0), (1024, 16, 2, 0), (4096, 32, 4, 0),
                                              (512, 4, 0, 1), (512, 8, 0, 2), (4096, 8, 0, 0)]:
            x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
            res = torch.randn(T, H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).to(torch.bfloat16)
            # reference: NCCL all-reduce (fp32 accumulate emulated by summing in fp32) + add + RMSNorm
            xs = x.float()
            dist.all_reduce(xs, group=tp.group)
            expect_res = xs.to(torch.bfloat16) + res
            expect = ref.rmsnorm(expect_res, w, 1e-5)
            view = buf.tensor[128:128 + T]                # a region that does not start at the buffer base
            view.copy_(x)
            my_res = res.clone()
            torch.cuda.synchronize()
            dist.barrier(group=tp.group)
            comm.fused_allreduce_add_rmsnorm_(view, my_res, w, 1e-5, max_ctas=ctas, mode=mode, rows_in_flight=rows_in_flight)
            torch.cuda.synchronize()
            dist.barrier(group=tp.group)
            rpr = T // world
            sl = slice(rank * rpr, (rank + 1) * rpr)
            got = view[sl] if mode == 1 else view
            want = expect[sl] if mode == 1 else expect
            # the reference's own check: allclose with atol = rtol = 4e-2 (artifact/figure_4_10/bench.py:243-244)
            def off(a, b):
                d = (a.float() - b.float()).abs()
                return int((d > 4e-2 + 4e-2 * b.float().abs()).sum().item()), d.max().item()
            bad, err = off(got, want)
            if bad:
                errors.append(f"fused T={T} ctas={ctas} mode={mode}: {bad} normed elements off, max err {err}")
            bad, rerr = off(my_res[sl], expect_res[sl])
            if bad:
                errors.append(f"fused T={T} ctas={ctas} mode={mode}: {bad} residual elements off, max err {rerr}")
            if mode != 1:
                # broadcast stores deliver one value everywhere: all ranks must hold identical bits
                chk = view.clone()
                dist.broadcast(chk, src=0, group=tp.group)
                if not torch.equal(chk, view):
                    errors.append(f"fused T={T}: ranks disagree bitwise")
        # stand-alone collectives
        for T, ctas in [(64, 4), (1024, 16)]:
            x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
            xs = x.float()
            dist.all_reduce(xs, group=tp.group)
            view = buf.tensor[:T]
            view.copy_(x)
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            comm.all_reduce_(view, ctas)
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            if (view.float() - xs).abs().max().item() > 4e-2 * max(1.0, xs.abs().max().item() / 8):
                errors.append(f"all_reduce T={T}")
            view.copy_(x)
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            comm.reduce_scatter_(view, ctas)
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            n = view.numel() // world
            if (view.view(-1)[rank * n:(rank + 1) * n].float() - xs.view(-1)[rank * n:(rank + 1) * n]).abs().max().item() > 0.1:
                errors.append(f"reduce_scatter T={T}")
            view.view(-1)[rank * n:(rank + 1) * n] = float(rank + 1)
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            comm.all_gather_(view, ctas)
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            for r in range(world):
                if not bool((view.view(-1)[r * n:(r + 1) * n] == float(r + 1)).all()):
                    errors.append(f"all_gather T={T} slice {r}")
            view.copy_(x)
            out = torch.empty_like(x)
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            comm.oneshot_all_reduce(view, out)
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            if (out.float() - xs).abs().max().item() > 4e-2 * max(1.0, xs.abs().max().item() / 8):
                errors.append(f"oneshot T={T}")
        try:
            ops.check_status()
        except Exception as e:
            errors.append(f"status: {e}")
    except Exception as e:
        import traceback
        errors.append(traceback.format_exc())
    torch.cuda.synchronize()
    dist.barrier(group=tp.group)
    try:
        buf.close()
    except Exception:
        import traceback
        errors.append(traceback.format_exc())
    pstate.destroy_distributed()
    assert not errors, "\n".join(errors)


@pytest.mark.parametrize("transport", ["multimem", "p2p", "native", "native-p2p"])
def test_fused_and_collectives_two_gpus(transport):
    _need_gpus(2)
    run_ranks(_comm_worker, 2, transport, timeout=300)


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("transport", ["multimem", "p2p"])
def test_fused_and_collectives_four_and_eight_gpus(world, transport):
    _need_gpus(world)
    run_ranks(_comm_worker, world, transport, timeout=300)


def _custom_ar_worker(rank, world):
    """The peer-to-peer all-reduce baseline and the package's own NCCL communicator against torch.distributed,
    on integer-valued data so that every path must agree bit for bit (the scheme of the reference's
    tests/distributed/test_custom_all_reduce.py:24-120), eagerly and replayed from a CUDA graph."""
    import torch.distributed as dist
    from tokenweave_b200 import ops
    from tokenweave_b200.parallel import state as pstate
    from tokenweave_b200.parallel.comm import TPCommunicator
    from tokenweave_b200.parallel.symm_mem import create_symmetric_buffer
    tp = pstate.init_distributed(rank, world, rank, "cuda")
    errors = []
    try:
        H = 8192
        buf = create_symmetric_buffer(2048, H, torch.bfloat16, tp)
        comm = TPCommunicator(buf, tp, wait_budget_ms=3000)
        assert comm.enable_pynccl(), "the ctypes NCCL communicator did not come up"
        g = torch.Generator(device="cuda").manual_seed(3 + rank)
        for enabled in (True, False):
            if enabled:
                comm.enable_custom_all_reduce()
            else:
                comm.custom_ar_enabled = False
            # one-shot (16 KB, 128 KB), two-shot (1 MB, 8 MB), beyond the limit (32 MB: NCCL)
            for T in (1, 8, 64, 512, 2048):
                x = torch.randint(0, 4, (T, H), device="cuda", generator=g).to(torch.bfloat16)
                want = x.clone()
                dist.all_reduce(want, group=tp.group)
                view = buf.tensor[:T]
                view.copy_(x)
                torch.cuda.synchronize(); dist.barrier(group=tp.group)
                comm.custom_all_reduce_(view)
                torch.cuda.synchronize(); dist.barrier(group=tp.group)
                if not torch.equal(view, want):
                    errors.append(f"custom all-reduce (enabled={enabled}) T={T}: differs from NCCL")
        comm.enable_custom_all_reduce()
        # the package's NCCL path, and both captured in one CUDA graph
        y = torch.randint(0, 4, (64, H), device="cuda", generator=g).to(torch.bfloat16)
        want = y.clone()
        dist.all_reduce(want, group=tp.group)
        z = y.clone()
        comm.nccl_all_reduce_(z)
        if not torch.equal(z, want):
            errors.append("pynccl all-reduce differs from torch.distributed")
        parts = torch.empty(world * 1024, device="cuda")
        comm.nccl_all_gather(parts, torch.full((1024,), float(rank), device="cuda"))
        if parts.view(world, 1024)[:, 7].tolist() != [float(r) for r in range(world)]:
            errors.append("pynccl all-gather order")
        view = buf.tensor[:64]
        z.copy_(y)
        view.copy_(y)
        torch.cuda.synchronize(); dist.barrier(group=tp.group)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            comm.custom_all_reduce_(view)
            comm.nccl_all_reduce_(z)
        for _ in range(3):
            view.copy_(y)
            z.copy_(y)
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            graph.replay()
            torch.cuda.synchronize(); dist.barrier(group=tp.group)
            if not (torch.equal(view, want) and torch.equal(z, want)):
                errors.append("graph replay of custom all-reduce / pynccl differs")
        ops.check_status()
        del graph
    except Exception:
        import traceback
        errors.append(traceback.format_exc())
    torch.cuda.synchronize()
    dist.barrier(group=tp.group)
    if comm.pynccl is not None:
        comm.pynccl.destroy()
    buf.close()
    pstate.destroy_distributed()
    assert not errors, "\n".join(errors)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_custom_all_reduce_and_pynccl_match_nccl_exactly(world):
    _need_gpus(world)
    run_ranks(_custom_ar_worker, world, timeout=300)


def test_bounded_wait_reports_instead_of_hanging():
    """A wait on a flag nobody sets runs out of its budget, the kernel returns and the host reads the
    status word; the context stays usable."""
    from tokenweave_b200 import ops
    from tokenweave_b200.ops import _native
    ops.reset_status()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    _native.call("tw_wait_probe", flag.data_ptr(), 200_000_000, ops.status_word().data_ptr(),
                 torch.cuda.current_stream().cuda_stream)
    with pytest.raises(ops.KernelStatusError) as ei:
        ops.check_status()
    assert ei.value.code & 2
    ops.reset_status()
    # the flag set before the wait: the kernel consumes it and reports nothing
    flag.fill_(1)
    _native.call("tw_wait_probe", flag.data_ptr(), 200_000_000, ops.status_word().data_ptr(),
                 torch.cuda.current_stream().cuda_stream)
    ops.check_status()
    assert int(flag.item()) == 0
    assert torch.ones(4, device="cuda").sum().item() == 4.0
