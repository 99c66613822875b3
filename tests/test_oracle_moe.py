"""Self-consistency of the MoE oracle: routing against an independent torch
statement of the reference's generator (tools/generate_gemma4_26b_moe_oracle.py:
86-91), permutation properties, and the ordered BF16 combine."""
import numpy as np
import torch

from oracle import codecs as C
from oracle import moe


def bf16_normal(shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).bfloat16().float().numpy()


def torch_route(scores, scales):
    p = torch.from_numpy(scores).softmax(-1, dtype=torch.float32)
    ids = p.argsort(dim=-1, descending=True, stable=True)[:, :8]
    w = p.gather(1, ids)
    w = w / w.sum(-1, keepdim=True) * torch.from_numpy(scales)[ids]
    ids, order = ids.sort(-1)
    return ids.int().numpy(), w.gather(1, order).numpy()


def test_route_matches_torch_statement():
    scores = bf16_normal((257, 128), 11)
    scales = bf16_normal((128,), 12, 0.1) + 1.0
    scales = C.bf16_round(scales)
    ids, w = moe.route(scores, scales)
    tids, tw = torch_route(scores, scales)
    assert np.array_equal(ids, tids)
    np.testing.assert_allclose(w, tw, rtol=2e-6, atol=0)


def test_route_ties_pick_lowest_ids():
    scores = np.zeros((17, 128), dtype=np.float32)
    ids, w = moe.route(scores, np.ones(128, dtype=np.float32))
    assert np.array_equal(ids, np.tile(np.arange(8, dtype=np.int32), (17, 1)))
    assert np.all(w == np.float32(0.125))


def test_route_patterns_from_reference_cases():
    """hot / distributed / uneven score patterns (generate_gemma4_26b_moe_oracle.py:70-81)."""
    for rows, mode in [(1, "hot"), (17, "distributed"), (129, "uneven")]:
        scores = torch.full((rows, 128), -4.0, dtype=torch.bfloat16)
        r = torch.arange(rows)
        starts = (r * 13) % 128 if mode == "distributed" else torch.where(r % 11 == 0, 120, 0) if mode == "uneven" else torch.zeros_like(r)
        ranks = torch.arange(8)
        scores.scatter_(1, (starts[:, None] + ranks) % 128, (5.0 - ranks * .125).bfloat16().expand(rows, 8))
        ids, _ = moe.route(scores.float().numpy(), np.ones(128, dtype=np.float32))
        expected = np.sort(((starts[:, None] + ranks) % 128).numpy(), axis=1)
        assert np.array_equal(ids, expected)


def test_permutation_properties():
    scores = bf16_normal((300, 128), 5)
    ids, _ = moe.route(scores, np.ones(128, dtype=np.float32))
    order, offsets = moe.permutation(ids)
    flat = ids.reshape(-1)
    assert np.array_equal(np.sort(order), np.arange(flat.size))
    assert offsets[0] == 0 and offsets[128] == flat.size
    for e in (0, 17, 127):
        seg = order[offsets[e]:offsets[e + 1]]
        assert np.all(flat[seg] == e) and np.all(np.diff(seg) > 0)   # stable


def test_combine_is_ordered_bf16_fold():
    rng = np.random.default_rng(3)
    tokens = 5
    down = C.bf16_round(rng.normal(0, 1, (tokens * 8, 2816)).astype(np.float32))
    weights = rng.random((tokens, 8)).astype(np.float32)
    inverse = rng.permutation(tokens * 8)
    out = C.bf16_to_f32(moe.combine(down, inverse, weights))
    t, d = 3, 1234
    s = np.float32(0)
    for j in range(8):
        prod = C.bf16_round(np.float32(down[inverse[t * 8 + j], d] * weights[t, j]))
        s = C.bf16_round(np.float32(s + prod))
    assert out[t, d] == s
