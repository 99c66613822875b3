"""NumPy restatement vs the reference's own scalar helpers compiled as host
code (oracle/_ref/libref_scalar.so, built by oracle/Makefile).  Skipped where
that library has not been built."""
import ctypes
from pathlib import Path

import numpy as np
import pytest

from oracle import codecs as C
from oracle import nvfp4

LIB = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libref_scalar.so"
pytestmark = pytest.mark.skipif(not LIB.exists(), reason="oracle/_ref not built")


@pytest.fixture(scope="module")
def ref():
    return ctypes.CDLL(str(LIB))


def _f32(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _inputs():
    rng = np.random.default_rng(7)
    special = np.array([0.0, -0.0, 448, 449, 463.9, 464, 480, 1e9, -1e9, 2.0 ** -10, 2.0 ** -9,
                        1.5 * 2.0 ** -9, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5, 6, 7, 100], dtype=np.float32)
    return np.concatenate([special, -special, rng.normal(0, 1, 200000).astype(np.float32),
                           (rng.normal(0, 1, 100000) * np.exp2(rng.integers(-12, 10, 100000))).astype(np.float32)])


def test_round_e4m3(ref):
    x = _inputs(); out = np.empty_like(x)
    ref.ref_round_e4m3(_f32(x), _f32(out), ctypes.c_long(x.size))
    assert np.array_equal(C.e4m3_round(x).view(np.uint32), out.view(np.uint32))


def test_round_e2m1(ref):
    x = _inputs(); out = np.empty_like(x)
    ref.ref_round_e2m1(_f32(x), _f32(out), ctypes.c_long(x.size))
    assert np.array_equal(C.e2m1_round(x).view(np.uint32), out.view(np.uint32))


def test_round_bf16(ref):
    x = _inputs(); out = np.empty(x.size, dtype=np.uint16)
    ref.ref_round_bf16(_f32(x), out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), ctypes.c_long(x.size))
    assert np.array_equal(C.bf16_bits(x), out)


@pytest.mark.parametrize("g", [1.0, 0.0737, 3.1e-5, 12.5])
def test_block_scale(ref, g):
    x = np.abs(_inputs()); out = np.empty_like(x)
    ref.ref_nvfp4_block_scale(_f32(x), ctypes.c_float(g), _f32(out), ctypes.c_long(x.size))
    assert np.array_equal(nvfp4.block_scale(x, g), out)
