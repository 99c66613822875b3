"""The allocation-free NVFP4 linear entry point (built-in scratch array).

Some users of this library cannot obtain device memory when they need a
projection -- an engine whose start-up gave all remaining HBM to its KV cache,
or a decode loop that must never stall in cudaMalloc -- and may have no scratch
region of their own to pass in.  gw_nvfp4_linear_static_scratch serves them.
This test calls it through the C ABI several times in a row (every kernel form
it can reach, larger problems before smaller ones so that stale bytes lie behind
them in the shared array) and requires the same BF16 bits as the plan-based
entry point with caller scratch, and agreement with the CPU oracle.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(gw, rows, k, n, seed, gelu=False):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn((n, k), generator=g) * 0.02).bfloat16().cuda()
    x = torch.randn((rows, 2 * k if gelu else k), generator=g).bfloat16().cuda()
    weight = gw.nvfp4_pack_weights(w, float(x.float().abs().max() / 2688))
    plan = gw.Nvfp4Plan(rows, k, n)
    scratch = torch.empty(plan.scratch_bytes(), dtype=torch.uint8, device="cuda")
    expected = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    plan.run(x, weight, expected, scratch, transform=1 if gelu else 0)
    return x, weight, expected


# (rows, K, N, seed, GeGLU input): weights on the lanes with and without the K split (<= 128 rows),
# tokens on the lanes (129..255 rows), the CTA-pair kernel (>= 256 rows), the fused GeGLU input;
# larger problems precede smaller ones so that stale packed rows and scale tiles lie behind them
CASES = [(64, 5376, 512, 1, False), (5, 256, 256, 2, False), (256, 4096, 256, 3, False), (200, 1024, 256, 4, False),
         (130, 256, 128, 5, False), (21, 704, 256, 6, True)]


def test_static_scratch_matches_plan_on_calls_in_a_row():
    import gewell_b200 as gw
    limit = gw.lib.gw_nvfp4_linear_static_scratch_limit()
    assert limit == 2 * 1024 * 1024
    problems = [_problem(gw, *case) for case in CASES]
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    outputs = []
    for (rows, k, n, _, gelu), (x, weight, _) in zip(CASES, problems):
        y = torch.full((rows * n + 64,), -5.0, dtype=torch.bfloat16, device="cuda")
        gw.nvfp4_linear_static_scratch(x, weight, k, n, y, transform=1 if gelu else 0)
        outputs.append(y)
    torch.cuda.synchronize()
    # this also collects the error word the built-in path reports its bounded waits into
    assert gw.kernel_error() == 0
    for (rows, k, n, _, gelu), (_, _, expected), y in zip(CASES, problems, outputs):
        assert torch.equal(y[:rows * n].reshape(rows, n), expected), f"rows={rows} K={k} N={n} gelu={gelu}"
        assert torch.all(y[rows * n:] == -5.0)
        assert torch.isfinite(expected.float()).all() and expected.float().abs().max() > 0


def test_static_scratch_against_the_cpu_oracle():
    """Not only equal to the plan path: one case straight against the faithful W4A4 oracle."""
    import gewell_b200 as gw
    from oracle import nvfp4 as onv
    from tests.gpu_helpers import assert_gemm_close, bits, device_weight_to_oracle
    rows, k, n = 48, 1024, 256
    x, weight, _ = _problem(gw, rows, k, n, 7)
    y = gw.nvfp4_linear_static_scratch(x, weight, k, n)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    expected = onv.linear_w4a4(x.float().cpu().numpy(), device_weight_to_oracle(weight, n, k), rcp_fn=gw.rcp_approx)
    assert_gemm_close(bits(y), expected, "static-scratch linear vs oracle")


def test_static_scratch_rejects_oversized_problems():
    import gewell_b200 as gw
    rows, k, n = 1024, 8192, 128          # 4 MiB of packed activations
    x = torch.zeros((rows, k), dtype=torch.bfloat16, device="cuda")
    w = gw.Nvfp4Weight(torch.zeros((n, k // 2), dtype=torch.uint8, device="cuda"),
                       torch.zeros(gw.nvfp4_scale_storage_bytes(n, k), dtype=torch.uint8, device="cuda"), 1.0, 1.0)
    with pytest.raises(gw.GewellInvalidArgument, match="exceed the built-in scratch"):
        gw.nvfp4_linear_static_scratch(x, w, k, n)
