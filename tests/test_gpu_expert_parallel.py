"""GPU tests of the expert-parallel building blocks through the C ABI:
gw_moe_run_sorted against the captured intermediates of the whole layer (one
GPU), and the 2-, 4- and 8-rank layer against the single-GPU layer (each needs
that many GPUs; skipped otherwise)."""
from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from tests.gpu_helpers import bf16_normal, bits  # noqa: E402

pytestmark = pytest.mark.gpu

E, H = 128, 2816


def _inputs(tokens: int, seed: int, skew: bool):
    x = bf16_normal((tokens, H), seed)
    logits = bf16_normal((tokens, E), seed + 1).float()
    if skew:
        ranks = torch.arange(1, E + 1, dtype=torch.float32)
        logits = logits + (ranks.pow(-1.2) / ranks.pow(-1.2).sum()).log()
    scales = (1.0 + 0.25 * torch.rand(E, generator=torch.Generator().manual_seed(seed + 2))).bfloat16()
    return x, logits.bfloat16(), scales


@pytest.fixture(scope="module")
def layer():
    import bench
    import gewell_b200 as gw
    experts = bench.build_experts(gw, torch, torch.device("cuda", 0))
    return gw, experts, gw.ExpertTable(experts)


@pytest.mark.parametrize("tokens", [33, 700])
def test_run_sorted_equals_layer_intermediates(layer, tokens):
    gw, _, table = layer
    x, scores, scales = (t.cuda() for t in _inputs(tokens, 40, False))
    ws = gw.MoeWorkspace(tokens)
    y = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
    ws.run(x, scores, scales, table, y, tokens)
    torch.cuda.synchronize()
    down = ws.down_capture()
    offsets, assignments = ws.offsets(), ws.sorted_assignments()
    n = 8 * tokens
    other = gw.MoeWorkspace(tokens)
    # (a) rows already in sorted order
    sorted_rows = gw.gather_rows(x, assignments, 8, n)
    out_a = torch.empty((n, H), dtype=torch.bfloat16, device="cuda")
    other.run_sorted(sorted_rows, offsets, 0, E, n, table, out_a)
    # (b) rows read through an index
    index = (assignments // 8).to(torch.int32)
    out_b = torch.empty((n, H), dtype=torch.bfloat16, device="cuda")
    other.run_sorted(x, offsets, 0, E, n, table, out_b, row_index=index)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert np.array_equal(bits(out_a), bits(down))
    assert np.array_equal(bits(out_b), bits(down))
    # the combine of those rows is the layer output
    _, _, inverse, weights = ws.routing_state(tokens)
    again = gw.moe_combine(out_b, inverse, weights, tokens)
    assert np.array_equal(bits(again), bits(y))


def test_absent_experts_are_accepted_and_validated(layer):
    gw, experts, _ = layer
    half = [ex if e < 64 else None for e, ex in enumerate(experts)]
    table = gw.ExpertTable(half)          # experts 64..127 live elsewhere
    tokens = 16
    x, _, _ = (t.cuda() for t in _inputs(tokens, 41, False))
    offsets = torch.zeros(65, dtype=torch.int32)
    offsets[1:] = torch.arange(1, 65) * 2            # two rows per local expert
    n = int(offsets[-1])
    rows = x.repeat(8, 1)[:n].contiguous()
    out = torch.empty((n, H), dtype=torch.bfloat16, device="cuda")
    ws = gw.MoeWorkspace(tokens)
    ws.run_sorted(rows, offsets.cuda(), 0, 64, n, table, out)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0 and torch.isfinite(out.float()).all()
    with pytest.raises(ValueError):
        ws.run_sorted(rows, offsets.cuda(), 100, 64, n, table, out)     # range leaves 0..128


def test_destination_tables_match_numpy(layer):
    gw, _, _ = layer
    from gewell_b200 import expert_parallel as ep
    rng = np.random.default_rng(3)
    for world in (1, 2, 8):
        owner = np.repeat(np.arange(world), E // world)
        rng.shuffle(owner)
        placement = ep.Placement(owner.tolist(), world)
        counts = rng.integers(0, 50, size=(world, E)).astype(np.int32)
        counts[rng.random(counts.shape) < 0.2] = 0
        per_rank = E // world
        totals = counts.sum(0)
        first = np.zeros(E, dtype=np.int64)
        for r in range(world):
            running = 0
            for e in placement.local_experts(r):
                first[e] = running
                running += totals[e]
        for rank in range(world):
            want_row0 = first + counts[:rank].sum(0)
            mine = placement.local_experts(rank)
            want_offsets = np.concatenate([[0], np.cumsum(totals[mine])])
            row0 = torch.zeros(E, dtype=torch.int32, device="cuda")
            offsets = torch.zeros(per_rank + 1, dtype=torch.int32, device="cuda")
            device_counts = torch.from_numpy(counts).cuda()
            device_physical = torch.tensor(placement.physical, dtype=torch.int32).cuda()
            segment_start = torch.zeros(world * per_rank, dtype=torch.int32, device="cuda")
            home_base = torch.zeros(world * per_rank, dtype=torch.int32, device="cuda")
            gw.ops._check(gw.lib.gw_moe_ep_tables(device_counts.data_ptr(), device_physical.data_ptr(), rank, world,
                                                  row0.data_ptr(), offsets.data_ptr(), segment_start.data_ptr(),
                                                  home_base.data_ptr(), torch.cuda.current_stream().cuda_stream))
            torch.cuda.synchronize()
            # the way home: segment of source s inside local expert j, and s's own sorted offset of that expert
            want_start = np.zeros((world, per_rank), dtype=np.int64)
            want_home = np.zeros((world, per_rank), dtype=np.int64)
            for j, e in enumerate(mine):
                want_start[:, j] = want_offsets[j] + np.concatenate([[0], np.cumsum(counts[:-1, e])])
                want_home[:, j] = [counts[s_, :e].sum() for s_ in range(world)]
            assert np.array_equal(segment_start.cpu().numpy().reshape(world, per_rank), want_start)
            assert np.array_equal(home_base.cpu().numpy().reshape(world, per_rank), want_home)
            assert np.array_equal(row0.cpu().numpy(), want_row0)
            assert np.array_equal(offsets.cpu().numpy(), want_offsets)


@pytest.mark.parametrize("tokens,send_home", [(40, False), (900, False), (40, True), (900, True)])
def test_record_path_on_one_rank_equals_layer(layer, tokens, send_home):
    """Dispatch into records, grouped GEMMs on the records, combine through the
    pointer table -- with this GPU as the only rank -- give the layer's output."""
    import ctypes
    gw, _, table = layer
    lib, check = gw.lib, gw.ops._check
    stream = torch.cuda.current_stream().cuda_stream
    x, scores, scales = (t.cuda() for t in _inputs(tokens, 60, True))
    ws = gw.MoeWorkspace(tokens)
    y = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
    ws.run(x, scores, scales, table, y, tokens)
    route_ws, expert_ws = gw.MoeWorkspace(tokens), gw.MoeWorkspace(tokens + 16)
    capacity = 8 * (tokens + 16)
    records = torch.full((capacity * 1584,), 0xFF, dtype=torch.uint8, device="cuda")    # stale bytes must not matter
    down = torch.empty((capacity, H), dtype=torch.bfloat16, device="cuda")
    route_ws.dispatch(scores, scales, tokens)
    offsets, _, _, _ = route_ws.routing_state(tokens)
    counts = (offsets[1:] - offsets[:-1]).contiguous()
    physical = torch.arange(E, dtype=torch.int32, device="cuda")
    dest_rank = torch.zeros(E, dtype=torch.int32, device="cuda")
    row0 = torch.zeros(E, dtype=torch.int32, device="cuda")
    local_offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    segment_start = torch.zeros(E, dtype=torch.int32, device="cuda")
    home_base = torch.zeros(E, dtype=torch.int32, device="cuda")
    check(lib.gw_moe_ep_tables(counts.data_ptr(), physical.data_ptr(), 0, 1, row0.data_ptr(), local_offsets.data_ptr(),
                               segment_start.data_ptr(), home_base.data_ptr(), stream))
    inverse_scales = (torch.ones(E) / torch.full((E,), 6.0 / 2688)).cuda()
    record_table = torch.tensor([records.data_ptr()], dtype=torch.int64, device="cuda")
    down_table = torch.tensor([down.data_ptr()], dtype=torch.int64, device="cuda")
    check(lib.gw_moe_ep_dispatch(route_ws._ws, x.data_ptr(), tokens, inverse_scales.data_ptr(), dest_rank.data_ptr(),
                                 row0.data_ptr(), record_table.data_ptr(), capacity, stream))
    if tokens <= 64:
        # the travelling records byte for byte: 1408 bytes of E2M1 and the 176 scale bytes in K order,
        # the row quantised with its expert's input scale (same recipe as moe.cu:254-304)
        from oracle import nvfp4 as onv
        torch.cuda.synchronize()
        host_records = records[:8 * tokens * 1584].reshape(8 * tokens, 1584).cpu().numpy()
        route_ws.rows = tokens
        order = route_ws.sorted_assignments().cpu().numpy()
        q = onv.quantize_activations(x.float().cpu().numpy()[order // 8], 6.0 / 2688, rcp_fn=gw.rcp_approx)
        assert np.array_equal(host_records[:, :1408], q.packed[:8 * tokens])
        assert np.array_equal(host_records[:, 1408:], q.scales_linear)
    out = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
    if send_home:
        returned = torch.full((8 * tokens, H), float("nan"), dtype=torch.bfloat16, device="cuda")
        returned_table = torch.tensor([returned.data_ptr()], dtype=torch.int64, device="cuda")
        check(lib.gw_moe_ep_run_experts(expert_ws._ws, records.data_ptr(), local_offsets.data_ptr(), 0, E, capacity,
                                        table.handle, None, segment_start.data_ptr(), home_base.data_ptr(),
                                        returned_table.data_ptr(), 8 * tokens, 1, stream))
        _, _, inverse, weights = route_ws.routing_state(tokens)
        check(lib.gw_moe_combine(returned.data_ptr(), inverse.data_ptr(), weights.data_ptr(), tokens, H, out.data_ptr(),
                                 stream))
    else:
        check(lib.gw_moe_ep_run_experts(expert_ws._ws, records.data_ptr(), local_offsets.data_ptr(), 0, E, capacity,
                                        table.handle, down.data_ptr(), None, None, None, 0, 1, stream))
        check(lib.gw_moe_ep_combine(route_ws._ws, tokens, dest_rank.data_ptr(), row0.data_ptr(), down_table.data_ptr(),
                                    capacity, out.data_ptr(), stream))
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert np.array_equal(local_offsets.cpu().numpy(), offsets.cpu().numpy())
    assert np.array_equal(bits(out), bits(y))
    # a buffer that is too small is reported, not overrun
    check(lib.gw_moe_ep_dispatch(route_ws._ws, x.data_ptr(), tokens, inverse_scales.data_ptr(), dest_rank.data_ptr(),
                                 row0.data_ptr(), record_table.data_ptr(), 8, stream))
    assert gw.kernel_error() >> 28 == 7


@pytest.mark.parametrize("distinct", [3, 128])
def test_dispatch_records_with_expert_input_scales(layer, distinct):
    """Every travelling record is quantised with the input scale of ITS expert.  With three scale values
    over the experts some of a token's eight copies repeat the scale of the copy before them (those leave
    from that copy's staged record), with 128 values none does; byte for byte against the oracle."""
    from oracle import nvfp4 as onv
    gw, _, _ = layer
    lib, check = gw.lib, gw.ops._check
    stream = torch.cuda.current_stream().cuda_stream
    tokens = 48
    x, scores, scales = (t.cuda() for t in _inputs(tokens, 63, True))
    route_ws = gw.MoeWorkspace(tokens)
    route_ws.dispatch(scores, scales, tokens)
    offsets, _, _, _ = route_ws.routing_state(tokens)
    counts = (offsets[1:] - offsets[:-1]).contiguous()
    physical = torch.arange(E, dtype=torch.int32, device="cuda")
    dest_rank = torch.zeros(E, dtype=torch.int32, device="cuda")
    row0 = torch.zeros(E, dtype=torch.int32, device="cuda")
    local_offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    check(lib.gw_moe_ep_tables(counts.data_ptr(), physical.data_ptr(), 0, 1, row0.data_ptr(), local_offsets.data_ptr(),
                               None, None, stream))
    input_scales = np.float32(6.0 / 2688) * (np.float32(1) + np.float32(0.03125) * (np.arange(E) % distinct).astype(np.float32))
    inverse_scales = torch.from_numpy((np.float32(1) / input_scales).astype(np.float32)).cuda()
    capacity = 8 * tokens
    records = torch.full((capacity * 1584,), 0xFF, dtype=torch.uint8, device="cuda")
    record_table = torch.tensor([records.data_ptr()], dtype=torch.int64, device="cuda")
    check(lib.gw_moe_ep_dispatch(route_ws._ws, x.data_ptr(), tokens, inverse_scales.data_ptr(), dest_rank.data_ptr(),
                                 row0.data_ptr(), record_table.data_ptr(), capacity, stream))
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    host_records = records.reshape(capacity, 1584).cpu().numpy()
    route_ws.rows = tokens
    order = route_ws.sorted_assignments().cpu().numpy()
    bounds = offsets.cpu().numpy()
    xf = x.float().cpu().numpy()
    checked = 0
    for e in range(E):
        first, last = int(bounds[e]), int(bounds[e + 1])
        if first == last:
            continue
        q = onv.quantize_activations(xf[order[first:last] // 8], float(input_scales[e]), rcp_fn=gw.rcp_approx)
        assert np.array_equal(host_records[first:last, :1408], q.packed[:last - first]), f"expert {e}"
        assert np.array_equal(host_records[first:last, 1408:], q.scales_linear[:last - first]), f"expert {e}"
        checked += last - first
    assert checked == capacity


def test_undersized_receive_capacity_is_reported_not_overrun(layer):
    """The group boundaries of a rank come from the other ranks' histograms.  If they describe more
    rows than the receive buffers were sized for, the grouped GEMMs must stop at the declared
    capacity and the combine must not read beyond it: guard rows behind the declared capacity stay
    untouched and the kernel error word reports the overflow."""
    gw, _, table = layer
    lib, check = gw.lib, gw.ops._check
    stream = torch.cuda.current_stream().cuda_stream
    tokens, declared = 48, 128            # 384 routed rows, buffers declared as 128 rows
    x, scores, scales = (t.cuda() for t in _inputs(tokens, 61, False))
    route_ws, expert_ws = gw.MoeWorkspace(tokens), gw.MoeWorkspace(tokens)
    route_ws.dispatch(scores, scales, tokens)
    offsets, _, _, _ = route_ws.routing_state(tokens)
    counts = (offsets[1:] - offsets[:-1]).contiguous()
    physical = torch.arange(E, dtype=torch.int32, device="cuda")
    dest_rank = torch.zeros(E, dtype=torch.int32, device="cuda")
    row0 = torch.zeros(E, dtype=torch.int32, device="cuda")
    local_offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    check(lib.gw_moe_ep_tables(counts.data_ptr(), physical.data_ptr(), 0, 1, row0.data_ptr(), local_offsets.data_ptr(),
                               None, None, stream))
    backing = 8 * tokens                  # real allocation: large enough that a missing clamp shows in the guards
    records = torch.zeros((backing * 1584,), dtype=torch.uint8, device="cuda")
    down = torch.full((backing, H), -9.0, dtype=torch.bfloat16, device="cuda")
    inverse_scales = (torch.ones(E) / torch.full((E,), 6.0 / 2688)).cuda()
    record_table = torch.tensor([records.data_ptr()], dtype=torch.int64, device="cuda")
    down_table = torch.tensor([down.data_ptr()], dtype=torch.int64, device="cuda")
    check(lib.gw_moe_ep_dispatch(route_ws._ws, x.data_ptr(), tokens, inverse_scales.data_ptr(), dest_rank.data_ptr(),
                                 row0.data_ptr(), record_table.data_ptr(), declared, stream))
    assert gw.kernel_error() >> 28 == 7
    assert torch.all(records[declared * 1584:] == 0), "dispatch wrote beyond the declared capacity"
    check(lib.gw_moe_ep_run_experts(expert_ws._ws, records.data_ptr(), local_offsets.data_ptr(), 0, E, declared,
                                    table.handle, down.data_ptr(), None, None, None, 0, 1, stream))
    assert gw.kernel_error() >> 28 == 7
    assert torch.all(down[declared:] == -9.0), "the grouped GEMMs wrote beyond the declared capacity"
    assert torch.isfinite(down[:declared].float()).all()
    out = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
    check(lib.gw_moe_ep_combine(route_ws._ws, tokens, dest_rank.data_ptr(), row0.data_ptr(), down_table.data_ptr(),
                                declared, out.data_ptr(), stream))
    assert gw.kernel_error() >> 28 == 7
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("tokens", [40, 900])
def test_activation_records_and_home_finish_on_one_rank(layer, tokens):
    """The exchange with the down projection at the tokens' home, this GPU being the only rank, through
    the C ABI: the travelling 416-byte activation records hold exactly the layer's quantised down input
    (352 bytes of E2M1, 44 scale bytes in K order), whichever kernel writes them (the gate/up epilogue
    for large batches, the export kernel for small ones); fetched back and finished with a table that
    holds only down matrices they give the layer's output bit for bit; undersized buffers are reported,
    not overrun."""
    from oracle import nvfp4 as onv
    gw, experts, table = layer
    lib, check = gw.lib, gw.ops._check
    stream = torch.cuda.current_stream().cuda_stream
    x, scores, scales = (t.cuda() for t in _inputs(tokens, 62, True))
    ws = gw.MoeWorkspace(tokens)
    ws.capture(True)
    y = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
    ws.run(x, scores, scales, table, y, tokens)
    torch.cuda.synchronize()
    activated = ws.activated_capture().float().cpu().numpy()             # [8 * tokens, 704] in sorted order
    record_bytes = int(lib.gw_moe_ep_activation_record_bytes())
    assert record_bytes == 416
    route_ws, expert_ws = gw.MoeWorkspace(tokens), gw.MoeWorkspace(tokens + 16)
    capacity = 8 * (tokens + 16)
    records = torch.full((capacity * 1584,), 0xFF, dtype=torch.uint8, device="cuda")
    act_records = torch.full((capacity * record_bytes + 64,), 0xEE, dtype=torch.uint8, device="cuda")
    route_ws.dispatch(scores, scales, tokens)
    offsets, _, _, _ = route_ws.routing_state(tokens)
    counts = (offsets[1:] - offsets[:-1]).contiguous()
    physical = torch.arange(E, dtype=torch.int32, device="cuda")
    dest_rank = torch.zeros(E, dtype=torch.int32, device="cuda")
    row0 = torch.zeros(E, dtype=torch.int32, device="cuda")
    local_offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    check(lib.gw_moe_ep_tables(counts.data_ptr(), physical.data_ptr(), 0, 1, row0.data_ptr(), local_offsets.data_ptr(),
                               None, None, stream))
    inverse_scales = (torch.ones(E) / torch.full((E,), 6.0 / 2688)).cuda()
    record_table = torch.tensor([records.data_ptr()], dtype=torch.int64, device="cuda")
    act_table = torch.tensor([act_records.data_ptr()], dtype=torch.int64, device="cuda")
    check(lib.gw_moe_ep_dispatch(route_ws._ws, x.data_ptr(), tokens, inverse_scales.data_ptr(), dest_rank.data_ptr(),
                                 row0.data_ptr(), record_table.data_ptr(), capacity, stream))
    check(lib.gw_moe_ep_run_gate_up(expert_ws._ws, records.data_ptr(), local_offsets.data_ptr(), 0, E, capacity,
                                    table.handle, act_records.data_ptr(), stream))
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    n = 8 * tokens
    host = act_records[:n * record_bytes].reshape(n, record_bytes).cpu().numpy()
    assert torch.all(act_records[capacity * record_bytes:] == 0xEE), "wrote beyond the record buffer"
    expected = onv.quantize_activations(activated, 16.0 / 2688, rcp_fn=gw.rcp_approx)     # the experts' down input scale
    assert np.array_equal(host[:, :352], expected.packed[:n])
    assert np.array_equal(host[:, 352:396], expected.scales_linear)
    # the home side: a table with the down matrices only
    home_table = gw.ExpertTable([(None, None, e[2]) for e in experts])
    out = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
    check(lib.gw_moe_ep_finish_at_home(route_ws._ws, tokens, dest_rank.data_ptr(), row0.data_ptr(), act_table.data_ptr(),
                                       capacity, home_table.handle, out.data_ptr(), stream))
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert np.array_equal(bits(out), bits(y))
    # a table without down matrices is refused; an undersized record buffer is reported, never read beyond
    with pytest.raises(gw.GewellInvalidArgument):
        check(lib.gw_moe_ep_finish_at_home(route_ws._ws, tokens, dest_rank.data_ptr(), row0.data_ptr(), act_table.data_ptr(),
                                           capacity, gw.ExpertTable([(e[0], e[1], None) for e in experts]).handle,
                                           out.data_ptr(), stream))
    check(lib.gw_moe_ep_finish_at_home(route_ws._ws, tokens, dest_rank.data_ptr(), row0.data_ptr(), act_table.data_ptr(),
                                       8, home_table.handle, out.data_ptr(), stream))
    assert gw.kernel_error() >> 28 == 7


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, placement_name: str, exchange: str, tokens: int, out_dir: str):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import bench
        import gewell_b200 as gw
        from gewell_b200 import expert_parallel as ep
        x, scores, scales = (t.to(device) for t in _inputs(tokens, 50, True))
        if placement_name == "balanced":
            histogram = torch.bincount(scores.float().topk(8, dim=1).indices.reshape(-1).cpu(), minlength=E)
            placement = ep.Placement.balanced(world, histogram.tolist())
        else:
            placement = getattr(ep.Placement, placement_name)(world)
        mine = placement.local_experts(rank)
        by_id = bench.build_experts(gw, torch, device, expert_ids=None if exchange == "home" else mine)
        by_position = [None] * E
        for e in mine:
            by_position[placement.physical[e]] = by_id[e]
        local = tokens // world
        if exchange in ("peer", "peer_pull", "peer_pull_nccl_sync", "home"):
            # histograms and barriers through mailboxes in peer memory, or ("..._nccl_sync") through NCCL
            moe = ep.PeerMemoryExpertParallelMoe(by_position, [6.0 / 2688] * E, rank, world, local, 8 * tokens,
                                                 placement=placement, send_home=exchange == "peer",
                                                 exchange="nccl" if exchange.endswith("nccl_sync") else "peer",
                                                 home_down=[w[2] for w in by_id] if exchange == "home" else None)
        else:
            backend = ep.DeviceBackend(by_position, local, 8 * tokens)
            moe = ep.ExpertParallelMoe(backend, rank, world, local, 8 * tokens, placement=placement)
        begin = rank * local
        for _ in range(3):                    # three steps: the mailboxes' two parities are both reused
            y = moe.run(x[begin:begin + local], scores[begin:begin + local], scales, local)
        torch.cuda.synchronize()
        assert gw.kernel_error() == 0
        np.save(os.path.join(out_dir, f"y{rank}.npy"), bits(y))
        if exchange != "nccl":
            moe.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,placement_name,exchange", [
    # one rank: the whole exchange machinery (records, mailboxes, activation records) on a single GPU
    (1, "contiguous", "peer_pull"), (1, "contiguous", "home"),
    (2, "contiguous", "nccl"), (2, "balanced", "nccl"), (2, "contiguous", "peer"), (2, "balanced", "peer"),
    (2, "balanced", "peer_pull"), (2, "balanced", "peer_pull_nccl_sync"), (2, "balanced", "home"), (2, "contiguous", "home"),
    (4, "interleaved", "home"), (8, "balanced", "home"),
    (4, "balanced", "peer_pull"), (4, "contiguous", "nccl"), (4, "interleaved", "peer"),
    (8, "balanced", "peer_pull"), (8, "interleaved", "nccl"), (8, "contiguous", "peer")])
def test_ranks_equal_single_gpu(layer, tmp_path, world, placement_name, exchange):
    """The expert-parallel layer over 2, 4 or 8 ranks (one process per GPU) returns the bits of the
    single-GPU layer, for every exchange implementation and placement."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    gw, _, table = layer
    tokens = 1536
    mp.spawn(_worker, args=(world, _free_port(), placement_name, exchange, tokens, str(tmp_path)), nprocs=world,
             join=True)
    x, scores, scales = (t.cuda() for t in _inputs(tokens, 50, True))
    ws = gw.MoeWorkspace(tokens)
    y = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
    ws.run(x, scores, scales, table, y, tokens)
    torch.cuda.synchronize()
    got = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(world)])
    expected = bits(y)
    mismatch = float(np.mean(got != expected))
    # the same kernels see the same rows; only the grouped-GEMM plan may differ with
    # the per-rank row count, and both plans accumulate the same products in FP32
    assert mismatch == 0.0, f"{mismatch:.2e} of the outputs differ between {world} ranks and 1 GPU"


def test_exchange_single_rank_and_missing_rank():
    """gw_moe_ep_exchange on one GPU: with one rank it hands back its own payload and counts its calls on the
    device; with a second rank that never publishes, the bounded wait runs out and the error word names it
    (the context stays usable)."""
    import gewell_b200 as gw
    lib = gw.lib
    size = int(lib.gw_moe_ep_mailbox_bytes())
    mailbox = torch.zeros(size, dtype=torch.uint8, device="cuda")
    other = torch.zeros(size, dtype=torch.uint8, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call in range(1, 4):
        payload = torch.arange(128, dtype=torch.int32, device="cuda") * call
        gathered = torch.full((1, 128), -1, dtype=torch.int32, device="cuda")
        table = torch.tensor([mailbox.data_ptr()], dtype=torch.int64, device="cuda")
        gw.ops._check(lib.gw_moe_ep_exchange(payload.data_ptr(), 128, table.data_ptr(), 0, 1, epoch.data_ptr(),
                                             gathered.data_ptr(), None))
        torch.cuda.synchronize()
        assert torch.equal(gathered[0], payload) and int(epoch.item()) == call
    assert gw.kernel_error() == 0
    # barrier only
    gw.ops._check(lib.gw_moe_ep_exchange(None, 0, table.data_ptr(), 0, 1, epoch.data_ptr(), None, None))
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0 and int(epoch.item()) == 4
    # rank 1 of 2 never arrives
    table = torch.tensor([mailbox.data_ptr(), other.data_ptr()], dtype=torch.int64, device="cuda")
    payload = torch.ones(4, dtype=torch.int32, device="cuda")
    gathered = torch.zeros((2, 4), dtype=torch.int32, device="cuda")
    gw.ops._check(lib.gw_moe_ep_exchange(payload.data_ptr(), 4, table.data_ptr(), 0, 2, epoch.data_ptr(),
                                         gathered.data_ptr(), None))
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0x90000000 | (1 << 8) | 0
    assert torch.equal(gathered[0], payload)                # its own values did arrive
    assert gw.kernel_error() == 0                           # the word is cleared on read; the context is intact
    with pytest.raises(gw.GewellInvalidArgument):
        gw.ops._check(lib.gw_moe_ep_exchange(payload.data_ptr(), 4, table.data_ptr(), 0, 9, epoch.data_ptr(),
                                             gathered.data_ptr(), None))
