"""GEMM fused with its collective (tw_gemm_rs_norm, tw_ag_gemm) on 2 GPUs, against the unfused sequence
GEMM -> NCCL all-reduce -> reference add+RMSNorm, over both transports, repeated calls included (the tile
counters return to zero and the shard epochs advance)."""
import math
import os

import pytest
import torch

from tw_testing import run_ranks

pytestmark = pytest.mark.gpu


def _worker(rank, world, transport):
    import torch.distributed as dist
    from tokenweave_b200 import ops
    from tokenweave_b200.ops import reference as ref
    from tokenweave_b200.parallel import state as pstate
    from tokenweave_b200.parallel.comm import TPCommunicator
    from tokenweave_b200.parallel.symm_mem import create_symmetric_buffer

    if transport == "p2p":
        os.environ["TW_DISABLE_NVLS"] = "1"
    tp = pstate.init_distributed(rank, world, rank, "cuda")
    errors = []
    try:
        H = 2048
        buf = create_symmetric_buffer(4096 + 512, H, torch.bfloat16, tp)
        comm = TPCommunicator(buf, tp, wait_budget_ms=3000)
        flags = create_symmetric_buffer(1, 8192, torch.bfloat16, tp, allow_multicast=False)
        comm.attach_flag_buffer(flags)
        gw = torch.Generator(device="cuda").manual_seed(11)
        norm_w = (1 + 0.1 * torch.randn(H, device="cuda", generator=gw)).to(torch.bfloat16)
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        # (T_pad, M, K of the row-parallel GEMM, N of the column-parallel GEMM, swiglu)
        cases = [(256, 256, 512, 1024, False), (1024, 1000, 1024, 1536, True), (64, 50, 256, 512, False),
                 (2048, 2048, 512, 2048, True), (1374, 1373, 512, 1024, False)]   # last: shards not aligned to tiles
        for rep in range(2):
            for (T, M, K, N2, swiglu) in cases:
                a = torch.randn(T, K, device="cuda", generator=g).to(torch.bfloat16)
                w1 = (torch.randn(H, K, device="cuda", generator=g) / math.sqrt(K)).to(torch.bfloat16)
                res0 = torch.randn(T, H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).to(torch.bfloat16)
                w2 = (torch.randn(2 * N2 if swiglu else N2, H, device="cuda", generator=gw) / math.sqrt(H)).to(torch.bfloat16)
                # reference
                part = ref.gemm(a[:M], w1).float()
                full = torch.zeros(T, H, device="cuda")
                full[:M] = part
                dist.all_reduce(full, group=tp.group)
                expect_res = full.to(torch.bfloat16) + res0
                expect_norm = ref.rmsnorm(expect_res, norm_w, 1e-5)
                expect_out = ref.gemm_swiglu(expect_norm[:M], w2) if swiglu else ref.gemm(expect_norm[:M], w2)
                rows = buf.tensor[256:256 + T]
                rows.zero_()
                res = res0.clone()
                out = torch.zeros(T, N2, device="cuda", dtype=torch.bfloat16)
                torch.cuda.synchronize(); dist.barrier(group=tp.group)
                assert comm.fused_gemm_available(rows)
                comm.gemm_rs_norm_(a, w1, rows, M, res, norm_w, 1e-5, comm_ctas=4)
                comm.ag_gemm(rows, w2, out, M, swiglu=swiglu, comm_ctas=4)
                torch.cuda.synchronize(); dist.barrier(group=tp.group)
                rpr = T // world
                sl = slice(rank * rpr, (rank + 1) * rpr)

                def off(x, y, tol=4e-2):
                    d = (x.float() - y.float()).abs()
                    return int((d > tol + tol * y.float().abs()).sum().item()), d.max().item()
                for name, got, want in (("residual shard", res[sl], expect_res[sl]), ("gathered norm", rows, expect_norm),
                                        ("consumer gemm", out[:M], expect_out)):
                    bad, err = off(got, want, 6e-2 if name == "consumer gemm" else 4e-2)
                    if bad:
                        errors.append(f"rep {rep} T={T} M={M} {name}: {bad} elements off, max err {err:.4f}")
        try:
            ops.check_status()
        except Exception as e:
            errors.append(f"status: {e}")
    except Exception:
        import traceback
        errors.append(traceback.format_exc())
    torch.cuda.synchronize()
    dist.barrier(group=tp.group)
    pstate.destroy_distributed()
    assert not errors, "\n".join(errors[:12])


@pytest.mark.parametrize("transport", ["multimem", "p2p"])
def test_fused_gemm_collectives_two_gpus(transport):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_worker, 2, transport, timeout=300)
