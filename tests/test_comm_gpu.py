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
