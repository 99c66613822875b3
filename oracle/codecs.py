"""Scalar number formats of the path, restated for NumPy arrays.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Formats and rounding rules follow the reference's scalar recipe:
  * E4M3FN, 127 finite magnitudes, subnormal step 2^-9, max 448, round to
    nearest even, finite saturation      -- src/weight_qdq_detail.cuh:61-63,
    tools/convert.py:39-62, tests/fp8_linear_test.cu:34-54
  * E2M1 levels {0,.5,1,1.5,2,3,4,6}, sign in bit 3, round to nearest even
    code, saturate at 6                  -- src/weight_qdq_detail.cuh:65-67,
    tools/convert.py:95-108, tests/nvfp4_linear_test.cu:33-66
  * BF16 round to nearest even of an FP32 value
                                         -- tools/safetensors_source.py:164-170

The encoders here work arithmetically (binade + quantum) rather than by table
search, so that they are an independent statement of the same rule; the table
decoders below are checked against them exhaustively in the CPU tests.
"""

from __future__ import annotations

import numpy as np

E2M1_LEVELS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_SIGNED = np.concatenate([E2M1_LEVELS, -E2M1_LEVELS]).astype(np.float32)     # code 8 decodes to -0.0


def _e4m3_table() -> np.ndarray:
    codes = np.arange(128, dtype=np.int64)
    exponent, mantissa = codes >> 3, codes & 7
    values = np.where(exponent == 0, mantissa * 2.0 ** -9,
                      (1.0 + mantissa / 8.0) * np.exp2(exponent - 7.0))
    values[127] = np.nan  # 0x7f is the only NaN pattern of E4M3FN
    return values.astype(np.float32)


E4M3_MAGNITUDES = _e4m3_table()          # index = code & 0x7f
E4M3_MAX = np.float32(448.0)
E2M1_MAX = np.float32(6.0)


# ----------------------------------------------------------------------------
# BF16
# ----------------------------------------------------------------------------

def bf16_bits(values) -> np.ndarray:
    """FP32 -> BF16 bit patterns (uint16), round to nearest even."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return rounded.astype(np.uint16)


def bf16_to_f32(bits) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def bf16_round(values) -> np.ndarray:
    """FP32 values rounded to the BF16 grid, returned as FP32."""
    return bf16_to_f32(bf16_bits(values))


# ----------------------------------------------------------------------------
# E4M3FN
# ----------------------------------------------------------------------------

def e4m3_decode(codes) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    magnitude = E4M3_MAGNITUDES[codes & 0x7F]
    return np.where(codes & 0x80, -magnitude, magnitude).astype(np.float32)


def e4m3_encode(values) -> np.ndarray:
    """FP32 -> E4M3FN code, nearest even, saturating to +/-448 (never NaN for
    finite input).  NaN input gives 0x7f like the satfinite device conversion."""
    values = np.asarray(values, dtype=np.float32)
    sign = np.signbit(values).astype(np.uint8) << 7
    magnitude = np.abs(values).astype(np.float64)
    nan = np.isnan(magnitude)
    magnitude = np.where(nan, 0.0, np.minimum(magnitude, 448.0))
    with np.errstate(divide="ignore"):
        binade = np.floor(np.log2(np.where(magnitude > 0, magnitude, 1.0)))
    binade = np.maximum(binade, -6.0)                 # subnormals share 2^-6's quantum
    quantum = np.exp2(binade - 3.0)
    rounded = np.rint(magnitude / quantum) * quantum   # np.rint rounds half to even
    # re-derive the code from the (representable) rounded magnitude
    with np.errstate(divide="ignore"):
        binade = np.floor(np.log2(np.where(rounded > 0, rounded, 1.0)))
    normal = rounded >= 2.0 ** -6
    exponent = np.where(normal, binade + 7.0, 0.0)
    mantissa = np.where(normal, (rounded / np.exp2(binade) - 1.0) * 8.0, rounded * 512.0)
    code = (exponent.astype(np.int64) << 3) | mantissa.astype(np.int64)
    code = np.where(nan, 0x7F, code).astype(np.uint8)
    return code | sign


def e4m3_round(values) -> np.ndarray:
    return e4m3_decode(e4m3_encode(values))


# ----------------------------------------------------------------------------
# E2M1
# ----------------------------------------------------------------------------

def e2m1_decode(codes) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    return np.take(E2M1_SIGNED, codes & 15)


def e2m1_encode(values) -> np.ndarray:
    """FP32 -> 4-bit E2M1 code (sign in bit 3), nearest even code, saturating."""
    values = np.asarray(values, dtype=np.float32)
    sign = np.signbit(values).astype(np.uint8) << 3
    magnitude = np.minimum(np.abs(values).astype(np.float64), 6.0)
    magnitude = np.where(np.isnan(magnitude), 6.0, magnitude)
    # quantum 0.5 below 2, 1 in [2,4), 2 in [4,6]
    quantum = np.where(magnitude < 2.0, 0.5, np.where(magnitude < 4.0, 1.0, 2.0))
    rounded = np.rint(magnitude / quantum) * quantum
    code = np.where(rounded < 2.0, rounded * 2.0,
                    np.where(rounded < 4.0, rounded + 2.0, rounded / 2.0 + 4.0))
    return code.astype(np.uint8) | sign


def e2m1_round(values) -> np.ndarray:
    return e2m1_decode(e2m1_encode(values))


def pack_nibbles(codes) -> np.ndarray:
    """[..., K] 4-bit codes -> [..., K/2] bytes, even element in the low nibble
    (include/gewell/nvfp4_linear.h:15-17)."""
    codes = np.asarray(codes, dtype=np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 15
    out[..., 1::2] = packed >> 4
    return out


# ----------------------------------------------------------------------------
# GeGLU with the two BF16 rounding boundaries  (src/bf16_activation.cuh:10-16)
# ----------------------------------------------------------------------------

def gelu_tanh_multiply_bf16(gate, up) -> np.ndarray:
    """bf16( bf16( 0.5*g*(1+tanh(0.79788456*(g+0.044715*g^3))) ) * up ), all
    intermediate arithmetic in FP32 in the reference's operation order."""
    g = np.asarray(gate, dtype=np.float32)
    u = np.asarray(up, dtype=np.float32)
    cube = g * g * g
    inner = np.float32(0.7978845608028654) * (g + np.float32(0.044715) * cube)
    activated = np.float32(0.5) * g * (np.float32(1.0) + np.tanh(inner).astype(np.float32))
    return bf16_round(bf16_round(activated) * u)
