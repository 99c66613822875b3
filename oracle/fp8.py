"""FP8 (E4M3FN) W8A8 linear layers on the CPU.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Restates:
  * the weight packer            tools/convert.py:49-92 (per tensor:
                                 weight_scale = amax/448); the per-output-channel
                                 variant applies the same codec per row
  * weight fake-quant (QDQ)      src/weight_qdq.cu:150-160,241-246
  * activation quantisation      src/fp8_linear.cu:33-52
  * the linear layer oracle      tests/fp8_linear_test.cu:95-117 (FP64 dot over
                                 decoded codes, times alpha or channel_scales[n])
  * the W8A16 host path          dequantise then FP32 matmul
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import codecs as C


@dataclass
class Weight:
    """Mirror of gewell::fp8::Weight (include/gewell/fp8_linear.h:17-24)."""
    data: np.ndarray              # [N, K] uint8 E4M3FN codes
    input_scale: float
    weight_scale: float
    channel_scales: np.ndarray | None = None   # [N] f32 alpha per output channel
    channel_weight_scales: np.ndarray | None = None  # [N] f32 dequant scale per row


def pack_weights(values: np.ndarray, input_scale: float = 1.0) -> Weight:
    """Per-tensor scale: weight_scale = f32(amax/448) (1 if all zero),
    code = e4m3(|x| / scale) (tools/convert.py:49-62,80-92)."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    assert np.all(np.isfinite(values)), "FP8 source contains nonfinite weights"
    amax = float(np.max(np.abs(values))) if values.size else 0.0
    scale = np.float32(amax / 448.0) if amax else np.float32(1)
    codes = C.e4m3_encode((values / scale).astype(np.float32))
    return Weight(codes, float(input_scale), float(scale))


def pack_weights_per_channel(values: np.ndarray, input_scale: float) -> Weight:
    """Joined projections: every output channel keeps its own scale
    scale_n = amax_n/448 and alpha_n = input_scale*scale_n
    (include/gewell/fp8_linear.h:21-23, 31b/sm120/fp8_projections.h:37-40)."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    amax = np.max(np.abs(values), axis=1).astype(np.float64)
    scale = np.where(amax > 0, (amax / 448.0), 1.0).astype(np.float32)
    codes = C.e4m3_encode((values / scale[:, None]).astype(np.float32))
    alpha = (np.float32(input_scale) * scale).astype(np.float32)
    return Weight(codes, float(input_scale), 1.0, alpha, scale)


def qdq(bits: np.ndarray) -> np.ndarray:
    """Static FP8 fake-quant of a flat BF16 tensor, bit patterns in and out:
    bf16( e4m3(x / s) * s ), s = amax/448 (src/weight_qdq.cu:150-160,241-246)."""
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    values = C.bf16_to_f32(bits)
    assert np.all(np.isfinite(values)), "non-finite BF16 value"
    amax = np.float32(np.max(np.abs(values))) if values.size else np.float32(0)
    if amax == 0:
        return bits.copy()
    scale = np.float32(amax / np.float32(448))
    normalized = (values / scale).astype(np.float32)
    return C.bf16_bits((C.e4m3_round(normalized) * scale).astype(np.float32))


def quantize_activations(x: np.ndarray, input_scale: float, gelu_width: int | None = None) -> np.ndarray:
    """e4m3_satfinite( fmul_rn(x, 1/input_scale) ) (src/fp8_linear.cu:33-52).
    With gelu_width=K the input is [M,2K] gate|up and GeGLU is applied first."""
    x = np.asarray(x, dtype=np.float32)
    if gelu_width is not None:
        x = C.gelu_tanh_multiply_bf16(x[:, :gelu_width], x[:, gelu_width:2 * gelu_width])
    inverse = np.float32(1) / np.float32(input_scale)
    with np.errstate(over="ignore"):
        return C.e4m3_encode((x * inverse).astype(np.float32))


def linear_w8a8(x: np.ndarray, weight: Weight, gelu: bool = False) -> np.ndarray:
    """tests/fp8_linear_test.cu:95-117.  Returns BF16 bits [M,N]."""
    k = weight.data.shape[1]
    codes = quantize_activations(x, weight.input_scale, k if gelu else None)
    acc = C.e4m3_decode(codes).astype(np.float64) @ C.e4m3_decode(weight.data).astype(np.float64).T
    if weight.channel_scales is not None:
        alpha = weight.channel_scales.astype(np.float32)[None, :]
    else:
        alpha = np.float32(np.float32(weight.input_scale) * np.float32(weight.weight_scale))
    return C.bf16_bits((acc * alpha.astype(np.float64) if isinstance(alpha, np.ndarray)
                        else acc * np.float64(alpha)).astype(np.float32))


def dequantize(weight: Weight) -> np.ndarray:
    """FP32 weights decode(code) * scale (tools/safetensors_source.py:197-198)."""
    scale = (weight.channel_weight_scales[:, None] if weight.channel_weight_scales is not None
             else np.float32(weight.weight_scale))
    return (C.e4m3_decode(weight.data) * scale).astype(np.float32)


def linear_w8a16(x: np.ndarray, weight: Weight) -> np.ndarray:
    """Host path of the north-star comparison: dequantise the weight, FP32
    matmul with the unquantised BF16 activations, BF16 out."""
    return C.bf16_bits(np.asarray(x, dtype=np.float32) @ dequantize(weight).T)
