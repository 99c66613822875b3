"""CPU tests of the artifact-entry checks and of bind_projection (no GPU: both are host code).  The
payloads are assembled, as the reference's artifact writer does (tools/gemma4_26b_mixed_artifact.py:
114-131), from outputs of the reference's own packers held in tests/golden/reference_packers.npz:
packed rows, zero padding rows, scale tiles from its swizzle_scale_chunk, the two FP32 globals."""
import ctypes
import struct

import numpy as np
import pytest

from gewell_b200 import _lib


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


@pytest.fixture(scope="module")
def golden(golden_dir):
    return np.load(golden_dir / "reference_packers.npz")


def nvfp4_entry(golden, name, rows_used=None):
    packed = golden[f"nvfp4_{name}_packed"]
    rows, half = packed.shape
    swizzled = golden[f"nvfp4_{name}_scales_swizzled"]
    weight_scale, input_scale = golden[f"nvfp4_{name}_globals"]
    return packed.tobytes() + swizzled.tobytes() + struct.pack("<ff", weight_scale, input_scale), rows, 2 * half


def check(lib, storage, rows, columns, payload):
    buffer = (ctypes.c_uint8 * len(payload)).from_buffer_copy(payload)
    status = lib.gw_validate_projection_entry(storage, rows, columns, buffer, len(payload))
    return status, lib.gw_last_error().decode()


@pytest.mark.parametrize("name", ["normal", "wide_range", "sparse"])
def test_entries_written_by_the_reference_packers_validate_and_bind(lib, golden, name):
    payload, rows, columns = nvfp4_entry(golden, name)
    assert lib.gw_projection_entry_bytes(_lib.STORAGE_NVFP4_W4A4, rows, columns) == len(payload)
    status, message = check(lib, _lib.STORAGE_NVFP4_W4A4, rows, columns, payload)
    assert status == _lib.GW_OK, message
    projection = _lib.Projection()
    host = (ctypes.c_uint8 * len(payload)).from_buffer_copy(payload)
    device_base = 0x7000_0000_0000            # any address: binding does not touch the device
    assert lib.gw_bind_projection(_lib.STORAGE_NVFP4_W4A4, rows, columns, host, device_base, len(payload),
                                  ctypes.byref(projection)) == _lib.GW_OK
    assert projection.nvfp4_data == device_base
    assert projection.nvfp4_scales == device_base + rows * columns // 2
    weight_scale, input_scale = golden[f"nvfp4_{name}_globals"]
    assert (projection.nvfp4_weight_scale, projection.nvfp4_input_scale) == (weight_scale, input_scale)
    assert (projection.input, projection.output, projection.physical_output) == (columns, rows, rows)
    # FP8 entry of the same tensor
    codes = golden[f"fp8_{name}_codes"]
    fp8_payload = codes.tobytes() + struct.pack("<ff", float(golden[f"fp8_{name}_scale"][0]), 0.125)
    status, message = check(lib, _lib.STORAGE_FP8_W8A8, rows, columns, fp8_payload)
    assert status == _lib.GW_OK, message


def test_padded_rows_sizes_and_rejections(lib, golden):
    # 704 x 2816 pads to 768 rows: size formula of tests/test_gemma4_26b_quantization.py:38-46
    assert lib.gw_projection_entry_bytes(_lib.STORAGE_NVFP4_W4A4, 704, 2816) == 768 * 2816 // 2 + 768 * 176 + 8
    assert lib.gw_projection_entry_bytes(_lib.STORAGE_FP8_W8A8, 704, 2816) == 704 * 2816 + 8
    assert lib.gw_projection_entry_bytes(_lib.STORAGE_BF16, 704, 2816) == 704 * 2816 * 2
    payload, rows, columns = nvfp4_entry(golden, "sparse")          # 128 x 64
    # the same tensor declared with 100 logical rows: rows 100..127 are padding and are not zero here
    status, message = check(lib, _lib.STORAGE_NVFP4_W4A4, 100, columns, payload)
    assert status == _lib.GW_INVALID_ARGUMENT and "padding" in message
    good = bytearray(payload)
    logical = 100 * columns // 2
    good[logical:rows * columns // 2] = bytes(rows * columns // 2 - logical)
    scales = np.frombuffer(bytes(good[rows * columns // 2:-8]), dtype=np.uint8).copy()
    r, c = np.meshgrid(np.arange(100, 128), np.arange(columns // 16), indexing="ij")
    scales[((c // 4) * 32 + r % 32) * 16 + (r // 32) * 4 + c % 4] = 0
    good[rows * columns // 2:-8] = scales.tobytes()
    status, message = check(lib, _lib.STORAGE_NVFP4_W4A4, 100, columns, bytes(good))
    assert status == _lib.GW_OK, message
    bad = bytearray(payload); bad[rows * columns // 2 + 5] = 0x7F
    assert check(lib, _lib.STORAGE_NVFP4_W4A4, rows, columns, bytes(bad))[1] == "invalid 26B NVFP4 block scale"
    bad = bytearray(payload); bad[-8:-4] = struct.pack("<f", float("inf"))
    assert check(lib, _lib.STORAGE_NVFP4_W4A4, rows, columns, bytes(bad))[1] == "invalid 26B global scales"
    bad = bytearray(payload); bad[-4:] = struct.pack("<f", 0.0)
    assert check(lib, _lib.STORAGE_NVFP4_W4A4, rows, columns, bytes(bad))[1] == "invalid 26B global scales"
    assert check(lib, _lib.STORAGE_NVFP4_W4A4, rows, columns, payload[:-1])[0] == _lib.GW_INVALID_ARGUMENT
    fp8 = bytes([0x38] * 15 + [0xFF]) + struct.pack("<ff", 0.25, 0.125)
    assert check(lib, _lib.STORAGE_FP8_W8A8, 1, 16, fp8)[1] == "nonfinite 26B FP8 payload"
    assert check(lib, 9, 1, 16, fp8)[1] == "invalid 26B storage type"


def test_policy_helper(lib):
    # include/gewell/nvfp4_policy.h:9-11
    assert lib.gw_nvfp4_fp4_activations(_lib.POLICY_ALWAYS, _lib.PHASE_DECODE) == 1
    assert lib.gw_nvfp4_fp4_activations(_lib.POLICY_PREFILL, _lib.PHASE_PREFILL) == 1
    assert lib.gw_nvfp4_fp4_activations(_lib.POLICY_PREFILL, _lib.PHASE_DECODE) == 0
