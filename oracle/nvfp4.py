"""NVFP4 (E2M1 values, E4M3 K16 block scales, FP32 global scale) on the CPU.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Restates, with NumPy:
  * the weight packer            tools/convert.py:95-137  (quantize_e2m1,
                                 quantize_nvfp4_tensor) and the scalar recipe
                                 src/weight_qdq_detail.cuh:61-82
  * the 128x4 scale tile layout  include/gewell/nvfp4_linear.h:35-56,
                                 tools/nvfp4_artifact.py:60-67,134-143
  * weight dequantisation        src/nvfp4_linear.cu:39-56,
                                 tools/safetensors_source.py:173-209
  * weight fake-quant (QDQ)      src/weight_qdq.cu:168-189,241-256
  * activation quantisation      src/nvfp4_linear.cu:61-116
  * the linear layer oracles     tests/nvfp4_linear_test.cu:263-293 (W4A4, FP64
                                 dot over decoded operands) and the W4A16 host
                                 path (dequantise, then FP32 matmul)
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import codecs as C

BLOCK = 16


# ----------------------------------------------------------------------------
# scale tile layout
# ----------------------------------------------------------------------------

def scale_storage_bytes(rows: int, width: int) -> int:
    """include/gewell/nvfp4_linear.h:35-38"""
    return ((rows + 127) // 128) * ((width + 63) // 64) * 512


def scale_offset(row, block, width):
    """Byte offset of the scale of (row, K16 block) in the tiled layout
    (include/gewell/nvfp4_linear.h:52-56).  Works on arrays."""
    row = np.asarray(row, dtype=np.int64)
    block = np.asarray(block, dtype=np.int64)
    return (((row // 128) * (width // 64) + block // 4) * 512
            + (row % 32) * 16 + ((row % 128) // 32) * 4 + block % 4)


def tile_scales(linear: np.ndarray, width: int) -> np.ndarray:
    """Linear [rows, width/16] scale bytes -> tiled storage, padding zero."""
    linear = np.asarray(linear, dtype=np.uint8)
    rows, blocks = linear.shape
    assert blocks == width // BLOCK and width % 64 == 0
    out = np.zeros(scale_storage_bytes(rows, width), dtype=np.uint8)
    r, b = np.meshgrid(np.arange(rows), np.arange(blocks), indexing="ij")
    out[scale_offset(r, b, width)] = linear
    return out


def untile_scales(tiled: np.ndarray, rows: int, width: int) -> np.ndarray:
    r, b = np.meshgrid(np.arange(rows), np.arange(width // BLOCK), indexing="ij")
    return np.asarray(tiled, dtype=np.uint8)[scale_offset(r, b, width)]


# ----------------------------------------------------------------------------
# weights
# ----------------------------------------------------------------------------

@dataclass
class Weight:
    """Mirror of gewell::nvfp4::Weight (include/gewell/nvfp4_linear.h:18-23)
    plus the shape, held on the host."""
    data: np.ndarray          # [N, K/2] uint8, even k in the low nibble
    scales: np.ndarray        # tiled E4M3 bytes, scale_storage_bytes(N, K)
    input_scale: float
    weight_scale: float
    rows: int                 # N (physical)
    width: int                # K


def weight_global_scale(values: np.ndarray) -> np.float32:
    """g = amax / (6*448), 1 for an all-zero tensor (tools/convert.py:118)."""
    amax = float(np.max(np.abs(values))) if values.size else 0.0
    return np.float32(amax / (6 * 448)) if amax else np.float32(1)


def pack_weights(values: np.ndarray, input_scale: float = 1.0,
                 weight_scale=None) -> Weight:
    """BF16-valued FP32 matrix [N,K] -> packed NVFP4 weight.

    tools/convert.py:111-137: block scale = e4m3(clip(bmax/(6 g), 2^-9, 448)),
    1 for an all-zero block; code = e2m1(x / (e4m3(scale) * g)) with the
    product formed in FP32 first."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    n, k = values.shape
    assert k % 64 == 0, "K must be divisible by 64"
    assert np.all(np.isfinite(values)), "NVFP4 source contains nonfinite weights"
    g = weight_global_scale(values) if weight_scale is None else np.float32(weight_scale)
    blocks = values.reshape(n, k // BLOCK, BLOCK)
    bmax = np.max(np.abs(blocks), axis=2)
    unrounded = bmax / (np.float32(6) * g)
    unrounded = np.where(bmax == 0, np.float32(1),
                         np.clip(unrounded, np.float32(1 / 512), np.float32(448))).astype(np.float32)
    scale_codes = C.e4m3_encode(unrounded)
    decoded = (C.e4m3_decode(scale_codes) * g).astype(np.float32)
    codes = C.e2m1_encode((blocks / decoded[:, :, None]).astype(np.float32)).reshape(n, k)
    return Weight(C.pack_nibbles(codes), tile_scales(scale_codes, k),
                  float(input_scale), float(g), n, k)


def pad_rows(weight: Weight, multiple: int = 128) -> Weight:
    """Zero-pad the output dimension to a multiple of 128 rows, as the 26B
    artifact does (projection.cu:37, tools/gemma4_26b_mixed_artifact.py:114-126):
    packed rows and scale bytes of the padding are zero."""
    physical = -(-weight.rows // multiple) * multiple
    if physical == weight.rows:
        return weight
    data = np.zeros((physical, weight.width // 2), dtype=np.uint8)
    data[:weight.rows] = weight.data
    linear = np.zeros((physical, weight.width // BLOCK), dtype=np.uint8)
    linear[:weight.rows] = untile_scales(weight.scales, weight.rows, weight.width)
    return Weight(data, tile_scales(linear, weight.width), weight.input_scale,
                  weight.weight_scale, physical, weight.width)


def decoded_weight_values(weight: Weight) -> tuple[np.ndarray, np.ndarray]:
    """(E2M1 values [N,K] f32, E4M3 block scales [N,K/16] f32) without the global."""
    values = C.e2m1_decode(C.unpack_nibbles(weight.data))
    scales = C.e4m3_decode(untile_scales(weight.scales, weight.rows, weight.width))
    return values, scales


def dequantize(weight: Weight) -> np.ndarray:
    """BF16 bit patterns [N,K] of bf16( e2m1 * (e4m3 * weight_scale) ), each
    product a single FP32 multiply (src/nvfp4_linear.cu:47-55)."""
    values, scales = decoded_weight_values(weight)
    multiplier = (scales * np.float32(weight.weight_scale)).astype(np.float32)
    product = (values.reshape(weight.rows, -1, BLOCK) * multiplier[:, :, None]).astype(np.float32)
    return C.bf16_bits(product.reshape(weight.rows, weight.width))


def block_scale(block_amax, global_scale) -> np.ndarray:
    """src/weight_qdq_detail.cuh:73-82 (nvfp4_block_scale)."""
    block_amax = np.asarray(block_amax, dtype=np.float32)
    g = np.float32(global_scale)
    unrounded = (block_amax / (np.float32(6) * g)).astype(np.float32)
    clamped = np.minimum(np.float32(448), np.maximum(np.float32(2.0 ** -9), unrounded))
    return np.where(block_amax == 0, np.float32(1), C.e4m3_round(clamped)).astype(np.float32)


def qdq(bits: np.ndarray) -> np.ndarray:
    """In-place style NVFP4 fake-quant of a flat BF16 tensor (bit patterns in,
    bit patterns out): src/weight_qdq.cu:168-189 with the global from :249-250.
    A tensor whose amax is zero is returned unchanged (:231-233)."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    values = C.bf16_to_f32(bits)
    assert values.size % BLOCK == 0
    assert np.all(np.isfinite(values)), "non-finite BF16 value"
    amax = np.float32(np.max(np.abs(values)))
    if amax == 0:
        return bits.copy()
    g = np.float32(amax / (np.float32(6) * np.float32(448)))
    blocks = values.reshape(-1, BLOCK)
    combined = (block_scale(np.max(np.abs(blocks), axis=1), g) * g).astype(np.float32)
    normalized = (blocks / combined[:, None]).astype(np.float32)
    out = (C.e2m1_round(normalized) * combined[:, None]).astype(np.float32)
    return C.bf16_bits(out.reshape(bits.shape))


# ----------------------------------------------------------------------------
# activations
# ----------------------------------------------------------------------------

def _ulp_neighbours(x: np.ndarray) -> list[np.ndarray]:
    x = np.asarray(x, dtype=np.float32)
    return [np.nextafter(x, np.float32(-np.inf)), x, np.nextafter(x, np.float32(np.inf))]


def rcp(x) -> np.ndarray:
    """Model of rcp.approx.ftz.f32: the correctly rounded FP32 reciprocal.  The
    hardware result is within one ulp of it; `quantize_activations_candidates`
    enumerates that uncertainty."""
    x = np.asarray(x, dtype=np.float32)
    with np.errstate(divide="ignore"):
        return (np.float32(1) / x).astype(np.float32)


@dataclass
class QuantizedActivations:
    packed: np.ndarray        # [padded_rows, K/2]
    scales_linear: np.ndarray  # [rows, K/16] E4M3 codes
    scales: np.ndarray        # tiled storage for `rows` rows
    rows: int
    padded_rows: int
    width: int


def quantize_activations(x: np.ndarray, input_scale: float, *, rcp6=None,
                         rcp_inverse=None, factor_delta: int = 0,
                         pad_to: int = 32, rcp_fn=None) -> QuantizedActivations:
    """BF16-valued FP32 activations [M,K] -> packed E2M1 + E4M3 K16 scales.

    src/nvfp4_linear.cu:61-116:
        inv    = 1 / input_scale                               (host FP32 divide)
        sf     = e4m3_satfinite( inv * (amax16 * rcp(6)) )
        factor = sf == 0 ? 0 : rcp( sf * rcp(inv) )
        code   = e2m1_rn( x * factor )
    `rcp6`, `rcp_inverse` override the two data-independent approximate
    reciprocals and `factor_delta` nudges the third by that many ulps; the
    defaults are the correctly rounded values.  `rcp_fn` replaces the reciprocal
    model altogether (the GPU tests pass the hardware instruction itself)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    assert k % 64 == 0
    inverse = np.float32(1) / np.float32(input_scale)
    rcp_ = rcp if rcp_fn is None else (lambda v: np.asarray(rcp_fn(np.asarray(v, dtype=np.float32)), dtype=np.float32))
    r6 = rcp_(np.float32(6)) if rcp6 is None else np.float32(rcp6)
    rinv = rcp_(inverse) if rcp_inverse is None else np.float32(rcp_inverse)
    blocks = x.reshape(m, k // BLOCK, BLOCK)
    amax = np.max(np.abs(blocks), axis=2).astype(np.float32)
    with np.errstate(over="ignore"):
        sf_code = C.e4m3_encode((inverse * (amax * r6).astype(np.float32)).astype(np.float32))
    sf = C.e4m3_decode(sf_code)
    denominator = (sf * rinv).astype(np.float32)
    factor = rcp_(np.where(sf == 0, np.float32(1), denominator))
    if factor_delta:
        step = np.float32(np.inf if factor_delta > 0 else -np.inf)
        for _ in range(abs(factor_delta)):
            factor = np.nextafter(factor, step)
    factor = np.where(sf == 0, np.float32(0), factor).astype(np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        scaled = (blocks * factor[:, :, None]).astype(np.float32)
    codes = C.e2m1_encode(scaled).reshape(m, k)
    padded_rows = -(-m // pad_to) * pad_to
    packed = np.zeros((padded_rows, k // 2), dtype=np.uint8)
    packed[:m] = C.pack_nibbles(codes)
    return QuantizedActivations(packed, sf_code, tile_scales(sf_code, k), m, padded_rows, k)


def quantize_activations_candidates(x, input_scale):
    """Every (packed, scale) outcome reachable when each approximate reciprocal
    is allowed to be one ulp either side of the correctly rounded value.
    Returns (packed_allowed[cand, M, K/2], scales_allowed[cand, M, K/16])."""
    inverse = np.float32(1) / np.float32(input_scale)
    packed, scales = [], []
    for r6 in _ulp_neighbours(rcp(np.float32(6))):
        for rinv in _ulp_neighbours(rcp(inverse)):
            for delta in (-1, 0, 1):
                q = quantize_activations(x, input_scale, rcp6=r6, rcp_inverse=rinv,
                                         factor_delta=delta)
                packed.append(q.packed[:q.rows])
                scales.append(q.scales_linear)
    return np.stack(packed), np.stack(scales)


def dequantized_activations(q: QuantizedActivations) -> np.ndarray:
    """Decoded activation values (E2M1 * E4M3 scale), without the global."""
    values = C.e2m1_decode(C.unpack_nibbles(q.packed[:q.rows]))
    scales = C.e4m3_decode(q.scales_linear)
    return (values.reshape(q.rows, -1, BLOCK) * scales[:, :, None]).reshape(q.rows, q.width).astype(np.float32)


# ----------------------------------------------------------------------------
# linear layers
# ----------------------------------------------------------------------------

def linear_w4a4_from_quantized(aq: np.ndarray, weight: Weight, logical_rows=None) -> np.ndarray:
    """tests/nvfp4_linear_test.cu:277-293: FP64 dot over decoded operands,
    times alpha = float(input_scale * weight_scale), rounded FP64->FP32->BF16.
    `aq` holds decoded activations [M,K].  Returns BF16 bits [M,N]."""
    values, scales = decoded_weight_values(weight)
    wq = (values.reshape(weight.rows, -1, BLOCK) * scales[:, :, None]).reshape(weight.rows, weight.width)
    n = weight.rows if logical_rows is None else logical_rows
    acc = aq.astype(np.float64) @ wq[:n].astype(np.float64).T
    alpha = np.float32(np.float32(weight.input_scale) * np.float32(weight.weight_scale))
    return C.bf16_bits((acc * np.float64(alpha)).astype(np.float32))


def linear_w4a4(x: np.ndarray, weight: Weight, gelu: bool = False, logical_rows=None, rcp_fn=None,
                gelu_fn=None) -> np.ndarray:
    """Faithful W4A4 oracle of nvfp4::Plan::run: quantise activations with the
    weight's input scale (optionally after GeGLU of [M,2K] gate|up slices,
    src/nvfp4_linear.cu:77-83), then the FP64 dot above."""
    x = np.asarray(x, dtype=np.float32)
    if gelu:
        k = weight.width
        x = (gelu_fn or C.gelu_tanh_multiply_bf16)(x[:, :k], x[:, k:2 * k])
    q = quantize_activations(x, weight.input_scale, rcp_fn=rcp_fn)
    return linear_w4a4_from_quantized(dequantized_activations(q), weight, logical_rows)


def linear_w4a16(x: np.ndarray, weight: Weight, logical_rows=None) -> np.ndarray:
    """The W4A16 host path: dequantise the weight to BF16
    (src/nvfp4_linear.cu:47-55), FP32 matmul with the BF16 activations, BF16 out
    (models/gemma4/26b_a4b/sm120/projection.cu:129-139)."""
    w = C.bf16_to_f32(dequantize(weight))
    n = weight.rows if logical_rows is None else logical_rows
    return C.bf16_bits(np.asarray(x, dtype=np.float32) @ w[:n].T)
