"""CPU paths of the small ops (activations, page copy / swap, partial-attention merge)."""
import math

import torch

from tokenweave_b200 import ops
from tokenweave_b200.ops import reference as ref


def test_activation_cpu_matches_torch():
    x = torch.randn(5, 32)
    assert torch.allclose(ops.activation(x, "gelu_and_mul"), torch.nn.functional.gelu(x[:, :16]) * x[:, 16:], atol=1e-6)
    assert torch.allclose(ops.activation(x, "quick_gelu"), x * torch.sigmoid(1.702 * x), atol=1e-6)
    assert ops.activation(x, "fatrelu_and_mul", param=0.5).shape == (5, 16)


def test_pages_cpu():
    cache = torch.arange(6 * 4, dtype=torch.float32).reshape(6, 4)
    ops.copy_pages(cache, torch.tensor([[0, 3], [1, 4]]))
    assert torch.equal(cache[3], cache[0]) and torch.equal(cache[4], cache[1])
    dst = torch.zeros(3, 4)
    ops.swap_pages(cache, dst, [(5, 0), (2, 2)])
    assert torch.equal(dst[0], cache[5]) and torch.equal(dst[2], cache[2]) and dst[1].abs().sum() == 0


def test_merge_cpu_is_exact_softmax_merge():
    H, D = 2, 8
    q, k, v = torch.randn(H, D), torch.randn(H, 12, D), torch.randn(H, 12, D)
    s = torch.einsum("hd,hkd->hk", q, k)
    full = torch.einsum("hk,hkd->hd", torch.softmax(s, -1), v)
    parts = []
    for sl in (slice(0, 5), slice(5, 12)):
        parts.append((torch.einsum("hk,hkd->hd", torch.softmax(s[:, sl], -1), v[:, sl]).unsqueeze(0),
                      torch.logsumexp(s[:, sl], -1).unsqueeze(1)))
    out, lse = ref.merge_attn_states(parts[0][0], parts[0][1], parts[1][0], parts[1][1])
    assert torch.allclose(out[0], full, atol=1e-5)
    assert torch.allclose(lse[:, 0], torch.logsumexp(s, -1), atol=1e-5)
    empty = torch.full((H, 1), -math.inf)
    out2, _ = ref.merge_attn_states(parts[0][0], parts[0][1], parts[1][0], empty)
    assert torch.allclose(out2, parts[0][0], atol=1e-6)


def test_gemm_plan_tables_answer_for_tuned_shapes_only():
    """The tuned plan tables (bf16 and e4m3) give a kernel and a tile width for the linear-layer shapes they were
    measured on, nothing for shapes far from any measurement, and keep the two operand types apart."""
    from tokenweave_b200.ops import gemm_table
    gemm_table.reload()
    for fp8 in (False, True):
        plan = gemm_table.lookup(4096, 8192, 1024, False, 0, fp8=fp8)       # o_proj of Llama-3.3-70B at TP = 8
        assert plan // 1000 in (1, 2) and 64 <= plan % 1000 <= 512 and plan % 1000 % 32 == 0
        sw = gemm_table.lookup(8192, 3584, 8192, True, 0, fp8=fp8)          # gate / up with the SwiGLU epilogue
        assert sw // 1000 in (1, 2) and sw % 1000 <= 256                     # no wide tiles with SwiGLU
        assert gemm_table.lookup(4096, 8200, 1000, False, 0, fp8=fp8) == 0  # never tuned: the cost model decides
        assert gemm_table.lookup(7, 8192, 1024, False, 0, fp8=fp8) == 0     # too far from any measured M
    gemm_table.set_enabled(False)
    try:
        assert gemm_table.lookup(4096, 8192, 1024, False, 0) == 0
    finally:
        gemm_table.set_enabled(True)


def test_int8_gemm_reference_is_exact_and_scaled():
    import torch
    from tokenweave_b200 import ops
    g = torch.Generator().manual_seed(0)
    a = torch.randint(-127, 128, (9, 64), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (5, 64), generator=g, dtype=torch.int8)
    raw = ops.gemm_int8(a, w, None, None)
    assert torch.equal(raw.float(), (a.long() @ w.long().t()).float().to(torch.bfloat16).float())
    a_s, w_s = torch.rand(9) + 0.5, torch.rand(5) + 0.5
    got = ops.gemm_int8(a, w, a_s, w_s, bias=torch.ones(5, dtype=torch.bfloat16))
    want = (a.long() @ w.long().t()).float() * a_s[:, None] * w_s[None, :] + 1.0
    torch.testing.assert_close(got.float(), want, rtol=1e-2, atol=1e-2)


def test_report_renders_the_committed_measurements():
    """artifact/report.py turns the benchmark CSVs into the figure tables (Markdown)."""
    import os
    import sys
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "artifact")
    sys.path.insert(0, root)
    import report
    text = report.report(os.path.join(root, "csvs"))
    assert "fused_microbench_tp8.csv" in text and "vs reference" in text
    assert "| 65536 | 1879.1 | 2295.2 | 1931.4 | 1.22x | 1.03x |" in text
    assert "throughput_llama70b_tp8_1024_64.csv" in text and "1.34x" in text
    rows = [{"model": "m", "tp": "2", "mode": "overlap", "tokens": "8", "latency_ms": "2.0", "device_ms": "1.0"},
            {"model": "m", "tp": "2", "mode": "no_ar", "tokens": "8", "latency_ms": "1.0", "device_ms": "0.5"}]
    assert "| 8 | 1.0 | 0.5 | 0.50x |" in report.prefill_table(rows)
