"""The 26B-A4B MoE layer (128 experts, top-8) on the CPU.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Restates:
  * routing      models/gemma4/26b_a4b/sm120/moe.cu:104-157 (select) and
                 tools/generate_gemma4_26b_moe_oracle.py:86-91: FP32 softmax,
                 eight winners by probability with the lower id winning ties,
                 renormalise times per-expert scale, sort the eight by id
  * permutation  tools/compare_gemma4_26b_moe.py:25-26: stable argsort of the
                 expert ids and searchsorted offsets (== moe.cu:158-182,477-488)
  * experts      moe.cu:254-352 (per projection activation quantisation with
                 the destination expert's input scale, alpha = in*weight scale),
                 GeGLU src/bf16_activation.cuh:10-16 (moe.cu:439-445)
  * combine      moe.cu:446-456: fold the eight slots in ascending expert id
                 with a BF16 rounding at the product and at every add
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import codecs as C
from . import fp8
from . import nvfp4

EXPERTS = 128
TOP_K = 8
HIDDEN = 2816
INTERMEDIATE = 704


@dataclass
class ExpertWeights:
    """Mirror of sm120::ExpertWeights{gate, up, down} (moe.cuh:11-13).  Each
    member carries its own storage, as in the reference: an oracle nvfp4.Weight
    (rows may be padded to 128), an fp8.Weight, or a BF16-valued FP32 matrix
    [N, K] for BF16 storage."""
    gate: object
    up: object
    down: object


def softmax_device_order(scores: np.ndarray) -> np.ndarray:
    """FP32 softmax over 128 logits with the device's reduction order
    (moe.cu:107-118): lane l holds elements l, l+32, l+64, l+96, adds its four
    exponentials in that order, then an xor-butterfly over the 32 lanes."""
    s = np.asarray(scores, dtype=np.float32).reshape(-1, 4, 32)
    maximum = s.max(axis=(1, 2), keepdims=True)
    e = np.exp((s - maximum).astype(np.float32)).astype(np.float32)
    lane = np.zeros((s.shape[0], 32), dtype=np.float32)
    for i in range(4):
        lane = (lane + e[:, i, :]).astype(np.float32)
    idx = np.arange(32)
    for offset in (16, 8, 4, 2, 1):
        lane = (lane + lane[:, idx ^ offset]).astype(np.float32)
    total = lane[:, :1, None]
    return (e / total).astype(np.float32).reshape(-1, EXPERTS)


def route(scores_bf16: np.ndarray, expert_scales_bf16: np.ndarray):
    """scores [T,128] and per-expert scales [128] as BF16-valued FP32.
    Returns (ids int32 [T,8] ascending, weights f32 [T,8])."""
    p = softmax_device_order(scores_bf16)
    # eight winners: higher probability first, lower id on ties
    order = np.argsort(-p, axis=1, kind="stable")[:, :TOP_K]
    chosen = np.take_along_axis(p, order, axis=1)
    s = chosen.copy()
    # moe.cu:146-147 pairwise tree ((p0+p4)+(p2+p6))+((p1+p5)+(p3+p7))
    s4 = (s[:, :4] + s[:, 4:]).astype(np.float32)
    s2 = (s4[:, :2] + s4[:, 2:]).astype(np.float32)
    total = (s2[:, :1] + s2[:, 1:]).astype(np.float32)
    scale = np.asarray(expert_scales_bf16, dtype=np.float32)[order]
    weights = ((chosen / total).astype(np.float32) * scale).astype(np.float32)
    by_id = np.argsort(order, axis=1, kind="stable")
    ids = np.take_along_axis(order, by_id, axis=1).astype(np.int32)
    weights = np.take_along_axis(weights, by_id, axis=1)
    return ids, weights


def permutation(ids: np.ndarray):
    """sorted_assignments [8T] (assignment = token*8+slot) and offsets [129]."""
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable").astype(np.int32)
    offsets = np.searchsorted(flat[order], np.arange(EXPERTS + 1)).astype(np.int32)
    return order, offsets


def _project(x: np.ndarray, weight, logical: int, mode: str, accumulate: str, rcp_fn=None) -> np.ndarray:
    """One expert projection; BF16-valued FP32 result [rows, logical].  BF16 weights: FP32 matmul,
    BF16 out (moe.cu:21-63,396-438); FP8 weights: the W8A8 oracle of the FP8 linear layer with the
    projection's own scales (moe.cu:187-251); NVFP4 weights by `mode`."""
    if isinstance(weight, np.ndarray):
        return C.bf16_round(np.asarray(x, dtype=np.float32) @ weight[:logical].T)
    if isinstance(weight, fp8.Weight):
        return C.bf16_to_f32(fp8.linear_w8a8(x, weight))[:, :logical]
    if mode == "w4a16":
        return C.bf16_to_f32(nvfp4.linear_w4a16(x, weight, logical))
    q = nvfp4.quantize_activations(x, weight.input_scale, rcp_fn=rcp_fn)
    aq = nvfp4.dequantized_activations(q)
    if accumulate == "f64":
        return C.bf16_to_f32(nvfp4.linear_w4a4_from_quantized(aq, weight, logical))
    values, scales = nvfp4.decoded_weight_values(weight)
    wq = (values.reshape(weight.rows, -1, 16) * scales[:, :, None]).reshape(weight.rows, weight.width)
    alpha = np.float32(np.float32(weight.input_scale) * np.float32(weight.weight_scale))
    return C.bf16_round(((aq @ wq[:logical].T).astype(np.float32) * alpha).astype(np.float32))


def forward(x_bf16: np.ndarray, scores_bf16: np.ndarray, expert_scales_bf16: np.ndarray,
            experts: list[ExpertWeights], mode: str = "w4a4", accumulate: str = "f64",
            capture: dict | None = None, rcp_fn=None, gelu_fn=None) -> np.ndarray:
    """Whole layer.  Inputs are BF16-valued FP32 arrays; returns BF16 bits
    [T, 2816].  `capture` (optional dict) receives ids, weights, order, offsets
    and the unfused intermediates gate_up / activated / down in sorted-row order
    (the reference's capture accessors, moe.cuh:38-40)."""
    x = np.asarray(x_bf16, dtype=np.float32)
    tokens = x.shape[0]
    ids, weights = route(scores_bf16, expert_scales_bf16)
    order, offsets = permutation(ids)
    n = TOP_K * tokens
    gate_up = np.zeros((n, 2 * INTERMEDIATE), dtype=np.float32)
    activated = np.zeros((n, INTERMEDIATE), dtype=np.float32)
    down = np.zeros((n, HIDDEN), dtype=np.float32)
    for e in range(EXPERTS):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if lo == hi:
            continue
        rows = x[order[lo:hi] // TOP_K]
        w = experts[e]
        g = _project(rows, w.gate, INTERMEDIATE, mode, accumulate, rcp_fn)
        u = _project(rows, w.up, INTERMEDIATE, mode, accumulate, rcp_fn)
        a = (gelu_fn or C.gelu_tanh_multiply_bf16)(g, u)
        gate_up[lo:hi, :INTERMEDIATE], gate_up[lo:hi, INTERMEDIATE:] = g, u
        activated[lo:hi] = a
        down[lo:hi] = _project(a, w.down, HIDDEN, mode, accumulate, rcp_fn)
    inverse = np.empty(n, dtype=np.int64)
    inverse[order] = np.arange(n)
    out = combine(down, inverse, weights)
    if capture is not None:
        capture.update(ids=ids, weights=weights, order=order, offsets=offsets,
                       gate_up=gate_up, activated=activated, down=down)
    return out


def combine(down: np.ndarray, inverse: np.ndarray, weights: np.ndarray) -> np.ndarray:
    """moe.cu:446-456.  down [8T,2816] BF16-valued; returns BF16 bits [T,2816]."""
    tokens = weights.shape[0]
    total = np.zeros((tokens, down.shape[1]), dtype=np.float32)
    for j in range(TOP_K):
        rows = down[inverse[np.arange(tokens) * TOP_K + j]]
        product = C.bf16_round((rows * weights[:, j:j + 1]).astype(np.float32))
        total = C.bf16_round((total + product).astype(np.float32))
    return C.bf16_bits(total)


# ----------------------------------------------------------------------------
# The W4A16 host path with the dequantised weights kept: what a CPU deployment of
# the reference's host path does (dequantise at load, FP32 matmul per step).  Used
# by the benchmark's CPU arm; same arithmetic as forward(mode="w4a16").
# ----------------------------------------------------------------------------

def dequantize_experts(experts: list[ExpertWeights]) -> list[tuple[np.ndarray, np.ndarray, np.ndarray]]:
    """BF16-rounded FP32 matrices (gate [704,2816], up [704,2816], down [2816,704]) of every
    expert: src/nvfp4_linear.cu:47-55 applied to each projection, padding rows dropped."""
    dense = []
    for w in experts:
        dense.append((C.bf16_to_f32(nvfp4.dequantize(w.gate))[:INTERMEDIATE],
                      C.bf16_to_f32(nvfp4.dequantize(w.up))[:INTERMEDIATE],
                      C.bf16_to_f32(nvfp4.dequantize(w.down))[:HIDDEN]))
    return dense


def forward_dequantized(x_bf16: np.ndarray, scores_bf16: np.ndarray, expert_scales_bf16: np.ndarray,
                        dense: list[tuple[np.ndarray, np.ndarray, np.ndarray]]) -> np.ndarray:
    """forward(mode="w4a16") over weights already dequantised by dequantize_experts."""
    x = np.asarray(x_bf16, dtype=np.float32)
    tokens = x.shape[0]
    ids, weights = route(scores_bf16, expert_scales_bf16)
    order, offsets = permutation(ids)
    n = TOP_K * tokens
    down = np.zeros((n, HIDDEN), dtype=np.float32)
    for e in range(EXPERTS):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if lo == hi:
            continue
        rows = x[order[lo:hi] // TOP_K]
        gate, up, down_w = dense[e]
        g = C.bf16_round(rows @ gate.T)
        u = C.bf16_round(rows @ up.T)
        a = C.gelu_tanh_multiply_bf16(g, u)
        down[lo:hi] = C.bf16_round(a @ down_w.T)
    inverse = np.empty(n, dtype=np.int64)
    inverse[order] = np.arange(n)
    return combine(down, inverse, weights)


def synthetic_packed_experts(seed: int = 4) -> list[ExpertWeights]:
    """128 experts of valid NVFP4 bytes drawn directly (uniform E2M1 codes, block scale codes in
    [2^-1, 2^2), one global scale that gives the weights a spread near 0.02), for timing the host
    path without running a packer over 760 M weights first.  Rows 704..767 of gate and up are the
    zero padding the artifact carries."""
    rng = np.random.default_rng(seed)
    experts = []
    for _ in range(EXPERTS):
        parts = []
        for rows, physical, width in ((INTERMEDIATE, 768, HIDDEN), (INTERMEDIATE, 768, HIDDEN), (HIDDEN, HIDDEN, INTERMEDIATE)):
            data = np.zeros((physical, width // 2), dtype=np.uint8)
            data[:rows] = rng.integers(0, 256, (rows, width // 2), dtype=np.uint8)
            linear = np.zeros((physical, width // nvfp4.BLOCK), dtype=np.uint8)
            linear[:rows] = rng.integers(0x30, 0x48, (rows, width // nvfp4.BLOCK), dtype=np.uint8)
            parts.append(nvfp4.Weight(data, nvfp4.tile_scales(linear, width), 6.0 / 2688, 0.02 / 3.0, physical, width))
        experts.append(ExpertWeights(*parts))
    return experts
