"""HostStagedMoe: layer passes with pinned host inputs and outputs, uploads and
downloads overlapped with the kernels.  Results must be bit-identical to
MoeWorkspace.run on device buffers, whatever the ring depth and however the
passes' row counts vary."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

H, E = 2816, 128


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the error raised without a device")
def test_host_staged_moe_needs_a_device():
    from gewell_b200.host_io import HostStagedMoe
    with pytest.raises(RuntimeError):
        HostStagedMoe(None, None, torch.ones(E, dtype=torch.bfloat16), 8, H)


@pytest.fixture(scope="module")
def layer():
    import gewell_b200 as gw
    from bench import build_experts                   # the benchmark's synthetic experts
    device = torch.device("cuda")
    experts = build_experts(gw, torch, device)
    table = gw.ExpertTable(experts)
    scales = (1.0 + 0.25 * torch.rand(E, device=device)).bfloat16()
    return gw, table, scales, experts


@pytest.mark.gpu
@pytest.mark.parametrize("depth", [1, 2, 3])
def test_host_staged_passes_match_device_runs(layer, depth):
    gw, table, scales, _ = layer
    device = torch.device("cuda")
    max_rows = 96
    ws = gw.MoeWorkspace(max_rows)
    runner = gw.HostStagedMoe(ws, table, scales, max_rows, H, depth=depth)
    g = torch.Generator().manual_seed(40 + depth)
    batches = []
    for rows in (96, 1, 40, 0, 77, 96, 13):
        x = torch.randn((max_rows, H), generator=g).bfloat16().pin_memory()
        s = torch.randn((max_rows, E), generator=g).bfloat16().pin_memory()
        y = torch.full((max_rows, H), 7.0, dtype=torch.bfloat16).pin_memory()
        batches.append((rows, x, s, y))
    tickets = [runner.submit(x, s, y, rows) for rows, x, s, y in batches]
    assert tickets == list(range(len(batches)))
    runner.wait_for(tickets[2])
    runner.synchronize()
    assert gw.kernel_error() == 0
    assert runner.h2d_bytes == sum(r for r, *_ in batches) * (H + E) * 2
    assert runner.d2h_bytes == sum(r for r, *_ in batches) * H * 2
    check = gw.MoeWorkspace(max_rows)
    for rows, x, s, y in batches:
        assert torch.all(y[rows:] == 7.0), "rows beyond the pass were written"
        if rows == 0:
            continue
        expected = torch.empty((rows, H), dtype=torch.bfloat16, device=device)
        check.run(x[:rows].to(device), s[:rows].to(device), scales, table, expected, rows)
        torch.cuda.synchronize()
        assert torch.equal(y[:rows], expected.cpu())


@pytest.mark.gpu
def test_host_staged_argument_checks(layer):
    gw, table, scales, _ = layer
    ws = gw.MoeWorkspace(8)
    runner = gw.HostStagedMoe(ws, table, scales, 8, H)
    x = torch.zeros((8, H), dtype=torch.bfloat16).pin_memory()
    s = torch.zeros((8, E), dtype=torch.bfloat16).pin_memory()
    y = torch.zeros((8, H), dtype=torch.bfloat16).pin_memory()
    with pytest.raises(ValueError):
        runner.submit(torch.zeros((8, H), dtype=torch.bfloat16), s, y, 8)      # not pinned
    with pytest.raises(ValueError):
        runner.submit(x, s, y, 9)                                               # more rows than the workspace
    with pytest.raises(ValueError):
        runner.submit(x.float().pin_memory(), s, y, 8)                          # wrong dtype
    with pytest.raises(ValueError):
        runner.wait_for(0)                                                      # nothing submitted
    with pytest.raises(ValueError):
        gw.HostStagedMoe(ws, table, scales, 8, H, depth=0)


@pytest.mark.gpu
@pytest.mark.parametrize("capture", [False, True])
def test_host_staged_custom_pass(layer, capture):
    """A caller's own layer pass (the expert-parallel layers use this hook) staged through the ring,
    launched eagerly or recorded once per ring slot and row count and replayed."""
    gw, table, scales, _ = layer
    device = torch.device("cuda")
    max_rows = 64
    ws = gw.MoeWorkspace(max_rows)
    calls = []

    def layer_pass(x, s, y, rows, stream):
        calls.append(rows)
        if rows:
            ws.run(x, s, scales, table, y, rows, stream=stream)

    warm = torch.zeros((max_rows, H), dtype=torch.bfloat16, device=device)
    ws.run(warm, torch.zeros((max_rows, E), dtype=torch.bfloat16, device=device), scales, table, torch.empty_like(warm), max_rows)
    torch.cuda.synchronize()
    runner = gw.HostStagedMoe(None, None, scales, max_rows, H, depth=2, run=layer_pass, capture=capture)
    g = torch.Generator().manual_seed(77)
    batches = []
    for rows in (64, 64, 64, 64, 9, 0, 9, 64):
        x = torch.randn((max_rows, H), generator=g).bfloat16().pin_memory()
        s = torch.randn((max_rows, E), generator=g).bfloat16().pin_memory()
        y = torch.full((max_rows, H), 7.0, dtype=torch.bfloat16).pin_memory()
        batches.append((rows, x, s, y))
        runner.submit(x, s, y, rows)
    runner.synchronize()
    assert gw.kernel_error() == 0
    # recorded passes call the hook once per (slot, rows); eager ones once per pass, zero rows included
    assert len(calls) == (len({(i % 2, r) for i, (r, *_) in enumerate(batches)}) if capture else len(batches))
    check = gw.MoeWorkspace(max_rows)
    for rows, x, s, y in batches:
        assert torch.all(y[rows:] == 7.0)
        if rows == 0:
            continue
        expected = torch.empty((rows, H), dtype=torch.bfloat16, device=device)
        check.run(x[:rows].to(device), s[:rows].to(device), scales, table, expected, rows)
        torch.cuda.synchronize()
        assert torch.equal(y[:rows], expected.cpu())
