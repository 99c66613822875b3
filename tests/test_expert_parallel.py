"""Host logic of the expert-parallel layer on CPU ranks (gloo, world size 2):
count exchange, split sizes, regrouping permutation, placement remapping and the
return path.  The CUDA library is replaced by a NumPy backend whose routing,
permutation and combine are the CPU oracle's and whose "expert MLP" is a cheap
function of (row, expert id), so a row that visits the wrong expert, or comes
home to the wrong slot, changes the result."""
from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from gewell_b200 import expert_parallel as ep  # noqa: E402
from oracle import codecs as C  # noqa: E402
from oracle import moe as omoe  # noqa: E402

WIDTH = 16


def expert_function(rows: np.ndarray, expert: int) -> np.ndarray:
    """Stand-in for the expert MLP: BF16-valued, different for every expert."""
    return C.bf16_round((rows * np.float32(1.0 + expert / 64.0) + np.float32(expert % 7)).astype(np.float32))


class HostBackend:
    def __init__(self, placement: ep.Placement):
        self.placement = placement

    def empty_rows(self, rows: int) -> torch.Tensor:
        return torch.zeros((rows, WIDTH), dtype=torch.float32)

    def route(self, scores, expert_scales, rows: int):
        ids, weights = omoe.route(scores.numpy()[:rows], expert_scales.numpy())
        order, offsets = omoe.permutation(ids)
        inverse = np.empty(order.size, dtype=np.int32)
        inverse[order] = np.arange(order.size, dtype=np.int32)
        return (torch.from_numpy(offsets), torch.from_numpy(order), torch.from_numpy(inverse),
                torch.from_numpy(weights.reshape(-1).copy()))

    def gather(self, x, index, divisor: int, rows: int, out):
        out[:rows] = x[(index[:rows].to(torch.int64) // divisor)]
        return out

    def experts(self, rows_in, row_index, local_offsets, first_expert: int, expert_count: int, total: int, out):
        offsets = local_offsets.tolist()
        for slot in range(expert_count):
            lo, hi = offsets[slot], offsets[slot + 1]
            if lo == hi:
                continue
            expert = self.placement.order[first_expert + slot]
            rows = rows_in[row_index[lo:hi].to(torch.int64)].numpy()
            out[lo:hi] = torch.from_numpy(expert_function(rows, expert))
        assert offsets[-1] == total
        return out

    def combine(self, down_rows, inverse, weights, rows: int, out):
        bits = omoe.combine(down_rows.numpy(), inverse.numpy().astype(np.int64), weights.numpy().reshape(rows, 8))
        out[:rows] = torch.from_numpy(C.bf16_to_f32(bits))
        return out


def single_process_reference(x: np.ndarray, scores: np.ndarray, scales: np.ndarray) -> np.ndarray:
    ids, weights = omoe.route(scores, scales)
    order, _ = omoe.permutation(ids)
    n = order.size
    down = np.zeros((n, WIDTH), dtype=np.float32)
    flat = ids.reshape(-1)
    for position, assignment in enumerate(order):
        down[position] = expert_function(x[assignment // 8][None, :], int(flat[assignment]))[0]
    inverse = np.empty(n, dtype=np.int64)
    inverse[order] = np.arange(n)
    return C.bf16_to_f32(omoe.combine(down, inverse, weights))


def make_inputs(tokens: int, seed: int, skew: bool):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((tokens, WIDTH), generator=g).bfloat16().float()
    scores = torch.randn((tokens, ep.EXPERTS), generator=g)
    if skew:
        ranks = torch.arange(1, ep.EXPERTS + 1, dtype=torch.float32)
        scores = scores + (ranks.pow(-1.2) / ranks.pow(-1.2).sum()).log()
    scores = scores.bfloat16().float()
    scales = (1.0 + 0.25 * torch.rand(ep.EXPERTS, generator=g)).bfloat16().float()
    return x, scores, scales


def _worker(rank: int, world: int, port: int, placement_name: str, tokens_per_rank: list[int], skew: bool, out_dir: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        placement = getattr(ep.Placement, placement_name)(world)
        total_tokens = sum(tokens_per_rank)
        x, scores, scales = make_inputs(total_tokens, 5, skew)
        begin = sum(tokens_per_rank[:rank])
        rows = tokens_per_rank[rank]
        layer = ep.ExpertParallelMoe(HostBackend(placement), rank, world, max(tokens_per_rank),
                                     8 * total_tokens, placement=placement)
        for _ in range(2):    # twice: buffers are reused between steps
            y = layer.run(x[begin:begin + rows], scores[begin:begin + rows], scales, rows)
        send, recv = layer.last_splits
        assert sum(send) == 8 * rows and sum(recv) == layer.last_layout.total
        np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
    finally:
        dist.destroy_process_group()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("placement_name,tokens_per_rank,skew", [
    ("contiguous", [24, 24], False),
    ("interleaved", [24, 24], True),
    ("contiguous", [5, 0], True),         # a rank without tokens still serves its experts
    ("interleaved", [1, 33], False),      # ragged
])
def test_two_ranks_match_single_process(tmp_path, placement_name, tokens_per_rank, skew):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), placement_name, tokens_per_rank, skew, str(tmp_path)),
             nprocs=world, join=True)
    x, scores, scales = make_inputs(sum(tokens_per_rank), 5, skew)
    expected = single_process_reference(x.numpy(), scores.numpy(), scales.numpy())
    got = np.concatenate([np.load(tmp_path / f"y{r}.npy")[:tokens_per_rank[r]] for r in range(world)])
    assert np.array_equal(got, expected)


def test_exchange_layout_against_brute_force():
    rng = np.random.default_rng(0)
    for sources, experts in ((1, 128), (2, 64), (8, 16), (4, 32)):
        counts = rng.integers(0, 5, size=(sources, experts))
        counts[rng.random(counts.shape) < 0.3] = 0
        total = int(counts.sum())
        layout = ep.exchange_layout(torch.from_numpy(counts.astype(np.int32)), total)
        arrival = [(s, e, k) for s in range(sources) for e in range(experts) for k in range(counts[s, e])]
        wanted = sorted(range(total), key=lambda j: (arrival[j][1], arrival[j][0], arrival[j][2]))
        assert layout.source_of_dest.tolist() == wanted
        assert [layout.dest_of_source[j].item() for j in wanted] == list(range(total))
        assert layout.local_offsets.tolist() == [0] + np.cumsum(counts.sum(0)).tolist()
    empty = ep.exchange_layout(torch.zeros((2, 64), dtype=torch.int32), 0)
    assert empty.total == 0 and empty.local_offsets.tolist() == [0] * 65


def test_placement_rules():
    for world in (1, 2, 4, 8):
        for p in (ep.Placement.contiguous(world), ep.Placement.interleaved(world)):
            assert sorted(p.order) == list(range(128))
            for r in range(world):
                mine = p.local_experts(r)
                assert len(mine) == 128 // world and mine == sorted(mine)
                assert all(p.owner[e] == r for e in mine)
                assert [p.physical[e] for e in mine] == list(range(r * p.per_rank, (r + 1) * p.per_rank))
    load = [1.0 / (e + 1) ** 1.2 for e in range(128)]
    balanced = ep.Placement.balanced(8, load)
    per_rank = [sum(load[e] for e in balanced.local_experts(r)) for r in range(8)]
    # optimum >= the heaviest expert plus the 15 lightest (every rank holds 16)
    assert max(per_rank) <= max(load[0] + sum(sorted(load)[:15]), sum(load) / 8) * 1.02
    assert sorted(balanced.order) == list(range(128))
    with pytest.raises(ValueError):
        ep.Placement([0] * 128, 2)
    with pytest.raises(ValueError):
        ep.Placement.contiguous(3)
