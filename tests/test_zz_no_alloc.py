"""The allocation-free NVFP4 linear entry point (built-in scratch array).

Some users of this library cannot obtain device memory when they need a
projection -- an engine whose start-up gave all remaining HBM to its KV cache,
or a decode loop that must never stall in cudaMalloc -- and may have no scratch
region of their own to pass in.  gw_nvfp4_linear_static_scratch serves them.
This test calls it through the C ABI twice in a row (a larger problem, then a
smaller one that leaves stale bytes behind it in the shared array) and requires
the same BF16 bits as the plan-based entry point with caller scratch.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(gw, rows, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn((n, k), generator=g) * 0.02).bfloat16().cuda()
    x = torch.randn((rows, k), generator=g).bfloat16().cuda()
    weight = gw.nvfp4_pack_weights(w, float(x.float().abs().max() / 2688))
    plan = gw.Nvfp4Plan(rows, k, n)
    scratch = torch.empty(plan.scratch_bytes(), dtype=torch.uint8, device="cuda")
    expected = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    plan.run(x, weight, expected, scratch)
    return x, weight, expected


def test_static_scratch_matches_plan_on_two_calls_in_a_row():
    import gewell_b200 as gw
    limit = gw.lib.gw_nvfp4_linear_static_scratch_limit()
    assert limit == 2 * 1024 * 1024
    cases = [(64, 5376, 512, 1), (5, 256, 256, 2)]
    problems = [_problem(gw, *case) for case in cases]
    torch.cuda.synchronize()
    outputs = []
    for (rows, k, n, _), (x, weight, _) in zip(cases, problems):
        y = torch.full((rows * n + 64,), -5.0, dtype=torch.bfloat16, device="cuda")
        gw.nvfp4_linear_static_scratch(x, weight, k, n, y)
        outputs.append(y)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    for (rows, k, n, _), (_, _, expected), y in zip(cases, problems, outputs):
        assert torch.equal(y[:rows * n].reshape(rows, n), expected), f"rows={rows} K={k} N={n}"
        assert torch.all(y[rows * n:] == -5.0)
        assert torch.isfinite(expected.float()).all() and expected.float().abs().max() > 0


def test_static_scratch_rejects_oversized_problems():
    import gewell_b200 as gw
    rows, k, n = 1024, 8192, 128          # 4 MiB of packed activations
    x = torch.zeros((rows, k), dtype=torch.bfloat16, device="cuda")
    w = gw.Nvfp4Weight(torch.zeros((n, k // 2), dtype=torch.uint8, device="cuda"),
                       torch.zeros(gw.nvfp4_scale_storage_bytes(n, k), dtype=torch.uint8, device="cuda"), 1.0, 1.0)
    with pytest.raises(gw.GewellInvalidArgument, match="exceed the built-in scratch"):
        gw.nvfp4_linear_static_scratch(x, w, k, n)
