"""The feed-forward block of a 26B-A4B layer around the MoE on the CPU: RMS norms, residual adds,
layer scalar.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Restates models/gemma4/26b_a4b/sm120/bf16_math.cuh:17-117 and the second half of the layer loop in
batched_executor.cu:250-286.  The reference builds this code with --fmad=false, so every product and sum
below is a separate FP32 rounding, which NumPy float32 arithmetic reproduces exactly.  The row reduction
follows the reference's fixed order:

  * the launch picks `lanes` logical lanes from the row count and the width (normalize_to, :86-95);
  * element i of a row belongs to lane (i // 4) % lanes and accumulator i % 4; an accumulator adds its
    squares by ascending i (norm :44-47, norm_parallel :69-71);
  * a lane's total is ((a0 + a1) + a2) + a3 (:48-49, :73-76); lanes fold in a halving tree (:51-54, :80-83);
  * inv = rsqrtf(total * (1 / width) + 1e-6) (:56, :84).

PARITY UNPINNED: the reference checks this code only through whole-layer captures against a fixture pack
of a torch run that is not part of its repository, and holds no golden vector for a norm by itself; the
functions below restate the kernel source line by line and are checked against nothing else.

rsqrtf is an approximate instruction: `rsqrt_fn` lets a test supply the device's values; the default is
the correctly rounded float32(1 / sqrt(x)), which differs from the hardware by at most a couple of FP32
ulps (a rare one-ulp flip after the BF16 rounding).
"""

from __future__ import annotations

import numpy as np

from . import codecs as C

RMS_EPSILON = np.float32(1e-6)      # include/gewell/models/gemma4/26b_a4b/model.h:26


def _floor_power_of_two(value: int) -> int:
    result = 1
    while result * 2 <= value:
        result *= 2
    return result


def reduction_lanes(rows: int, width: int) -> int:
    """normalize_to (bf16_math.cuh:86-95)."""
    dim = _floor_power_of_two(min(512, max(1, width // 4)))
    height = _floor_power_of_two(min(16, max(1, rows)))
    return min(dim, 512 // height)


def _host_rsqrt(values: np.ndarray) -> np.ndarray:
    return (np.float32(1) / np.sqrt(values.astype(np.float64))).astype(np.float32)


def inverse_rms(x: np.ndarray, lanes: int, rsqrt_fn=None) -> np.ndarray:
    """x: FP32 [rows, width] (BF16 values).  Returns FP32 [rows]."""
    x = np.asarray(x, dtype=np.float32)
    rows, width = x.shape
    square = x * x                                            # one FP32 rounding per product
    group = 4 * lanes
    steps = -(-width // group)
    padded = np.zeros((rows, steps * group), dtype=np.float32)    # + 0.0 leaves an accumulator unchanged
    padded[:, :width] = square
    padded = padded.reshape(rows, steps, lanes, 4)
    partial = np.zeros((rows, lanes, 4), dtype=np.float32)
    for step in range(steps):
        partial = partial + padded[:, step]
    total = ((partial[..., 0] + partial[..., 1]) + partial[..., 2]) + partial[..., 3]
    count = lanes
    while count > 1:
        count //= 2
        total = total[:, :count] + total[:, count:2 * count]
    mean = total[:, 0] * (np.float32(1) / np.float32(width)) + RMS_EPSILON
    return (rsqrt_fn or _host_rsqrt)(mean.astype(np.float32)).astype(np.float32)


def rms_norm(x: np.ndarray, weight, launch_rows: int | None = None, rsqrt_fn=None) -> np.ndarray:
    """bf16_math::normalize: FP32 [rows, width] of BF16 values in, BF16 values (FP32) out."""
    x = np.asarray(x, dtype=np.float32)
    lanes = reduction_lanes(launch_rows or x.shape[0], x.shape[1])
    normal = x * inverse_rms(x, lanes, rsqrt_fn)[:, None]
    if weight is None:
        return C.bf16_round(normal)
    return C.bf16_round(normal * np.asarray(weight, dtype=np.float32)[None, :])


def rms_norm_feedforward(x, shared_weight, router_weight, expert_weight, rsqrt_fn=None):
    """bf16_math::normalize_feedforward (FeedForwardNormOutput, :25-37): (shared, router, expert)."""
    x = np.asarray(x, dtype=np.float32)
    width = x.shape[1]
    normal = x * inverse_rms(x, reduction_lanes(x.shape[0], width), rsqrt_fn)[:, None]
    shared = C.bf16_round(normal * np.asarray(shared_weight, dtype=np.float32)[None, :])
    expert = C.bf16_round(normal * np.asarray(expert_weight, dtype=np.float32)[None, :])
    weighted = C.bf16_round(C.bf16_round(normal) * np.asarray(router_weight, dtype=np.float32)[None, :])
    router_scale = np.float32(1) / np.sqrt(np.float32(width))
    router = C.bf16_round(weighted * router_scale)
    return shared, router, expert


def add(a, b) -> np.ndarray:
    with np.errstate(over="ignore"):                   # FP32 overflow gives inf, as on the device
        return C.bf16_round(np.asarray(a, dtype=np.float32) + np.asarray(b, dtype=np.float32))


def scale(x, scalar) -> np.ndarray:
    return C.bf16_round(np.asarray(x, dtype=np.float32) * np.float32(scalar))


def tail(hidden, shared_mlp, routed, norm_shared, norm_routed, norm_sum, layer_scalar, rsqrt_fn=None) -> np.ndarray:
    """batched_executor.cu:260,278-285."""
    shared = rms_norm(shared_mlp, norm_shared, rsqrt_fn=rsqrt_fn)
    branch = rms_norm(routed, norm_routed, rsqrt_fn=rsqrt_fn)
    shared = add(shared, branch)
    branch = rms_norm(shared, norm_sum, rsqrt_fn=rsqrt_fn)
    return scale(add(hidden, branch), layer_scalar)
