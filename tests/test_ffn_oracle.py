"""CPU checks of the feed-forward-block oracle (oracle/ffn.py) and of the launch rule the library shares
with it (host code: no GPU)."""
import numpy as np

from gewell_b200 import _lib
from oracle import codecs as C
from oracle import ffn as offn


def test_reduction_lanes_rule_matches_library():
    lib = _lib.load()
    for rows in (1, 2, 3, 4, 5, 8, 15, 16, 17, 4096):
        for width in (8, 16, 64, 256, 512, 2048, 2816, 16384):
            assert lib.gw_rms_norm_reduction_lanes(rows, width) == offn.reduction_lanes(rows, width)
    # the layer's width: 512 lanes for one row down to 32 from 16 rows on (bf16_math.cuh:86-95)
    assert [offn.reduction_lanes(r, 2816) for r in (1, 2, 4, 8, 16, 8192)] == [512, 256, 128, 64, 32, 32]


def test_norm_oracle_against_float64():
    """The ordered FP32 reduction stays within FP32 rounding of the exact mean, and every output within one
    BF16 ulp of the exactly computed norm."""
    rng = np.random.default_rng(0)
    x = C.bf16_round(rng.standard_normal((9, 2816)).astype(np.float32) * 3)
    w = C.bf16_round(1 + 0.2 * rng.standard_normal(2816).astype(np.float32))
    for rows in (1, 4, 9):
        inv = offn.inverse_rms(x[:rows], offn.reduction_lanes(rows, 2816))
        exact = 1 / np.sqrt((x[:rows].astype(np.float64) ** 2).mean(axis=1) + 1e-6)
        assert np.max(np.abs(inv / exact - 1)) < 5e-7
        y = offn.rms_norm(x[:rows], w)
        reference = x[:rows].astype(np.float64) * exact[:, None] * w[None, :]
        assert np.max(np.abs(y - reference) / np.maximum(np.abs(reference), 1e-30)) < 2.0 ** -7


def test_feedforward_outputs_and_tail_compose():
    rng = np.random.default_rng(1)
    x = C.bf16_round(rng.standard_normal((3, 2816)).astype(np.float32))
    ws, wr, we = (C.bf16_round(1 + 0.1 * rng.standard_normal(2816).astype(np.float32)) for _ in range(3))
    shared, router, expert = offn.rms_norm_feedforward(x, ws, wr, we)
    assert np.array_equal(shared, offn.rms_norm(x, ws)) and np.array_equal(expert, offn.rms_norm(x, we))
    unweighted = offn.rms_norm(x, None)
    expected = C.bf16_round(C.bf16_round(unweighted * wr) * (np.float32(1) / np.sqrt(np.float32(2816))))
    assert np.array_equal(router, expected)
    hidden = C.bf16_round(rng.standard_normal((3, 2816)).astype(np.float32))
    out = offn.tail(hidden, shared, expert, ws, wr, we, 0.5)
    summed = offn.add(offn.rms_norm(shared, ws), offn.rms_norm(expert, wr))
    assert np.array_equal(out, offn.scale(offn.add(hidden, offn.rms_norm(summed, we)), 0.5))
