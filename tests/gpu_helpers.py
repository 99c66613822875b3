"""Shared helpers of the GPU parity tests: seeded inputs, transfers between
torch device tensors and the NumPy oracle, and the error metrics of the
acceptance criteria."""
from __future__ import annotations

import numpy as np
import torch

from oracle import codecs as C
from oracle import nvfp4 as onv


def bf16_normal(shape, seed: int, std: float = 1.0) -> torch.Tensor:
    """CPU BF16 tensor ~ N(0, std), from torch.Generator(seed) so that the
    oracle and the device see identical bits."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)


def to_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def device_weight_to_oracle(w, rows: int, width: int) -> onv.Weight:
    """gewell_b200.Nvfp4Weight (device) -> oracle Weight (host)."""
    return onv.Weight(w.data.cpu().numpy().reshape(rows, width // 2), w.scales.cpu().numpy(),
                      w.input_scale, w.weight_scale, rows, width)


def oracle_weight_to_device(w: onv.Weight, device="cuda"):
    import gewell_b200 as gw
    return gw.Nvfp4Weight(torch.from_numpy(w.data.copy()).to(device), torch.from_numpy(w.scales.copy()).to(device),
                          w.input_scale, w.weight_scale)


def error_metrics(actual_bits: np.ndarray, expected_bits: np.ndarray) -> dict:
    a = C.bf16_to_f32(actual_bits).astype(np.float64)
    e = C.bf16_to_f32(expected_bits).astype(np.float64)
    diff = np.abs(a - e)
    return {
        "max_abs": float(diff.max()) if diff.size else 0.0,
        "max_ref": float(np.abs(e).max()) if e.size else 0.0,
        "rel_fro": float(np.linalg.norm(a - e) / max(np.linalg.norm(e), 1e-30)),
        "mismatch": float(np.mean(actual_bits != expected_bits)) if diff.size else 0.0,
        "finite": bool(np.isfinite(a).all()),
    }


def assert_gemm_close(actual_bits, expected_bits, what=""):
    """Acceptance bound of the path: max abs error <= 1e-2 * max|Y_ref| or
    relative Frobenius error <= 5e-3, and all outputs finite."""
    m = error_metrics(actual_bits, expected_bits)
    assert m["finite"], f"{what}: non-finite output"
    ok = m["max_abs"] <= 1e-2 * m["max_ref"] or m["rel_fro"] <= 5e-3
    assert ok, f"{what}: {m}"
    return m


def assert_reference_tolerance(actual_bits, expected_bits, what=""):
    """Element-wise bound used by the reference's own linear tests
    (tests/nvfp4_linear_test.cu:289-290): |got-ref| <= max(0.008*|ref|, 0.001)."""
    a = C.bf16_to_f32(actual_bits).astype(np.float64)
    e = C.bf16_to_f32(expected_bits).astype(np.float64)
    bound = np.maximum(0.008 * np.abs(e), 0.001)
    bad = np.abs(a - e) > bound
    assert np.isfinite(a).all(), f"{what}: non-finite output"
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} outside tolerance; worst {np.abs(a - e).max()}"
