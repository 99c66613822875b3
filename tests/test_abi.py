"""The C-ABI library loads on a machine without a GPU and exports every
symbol that include/gewell_b200.h (the drop-in surface) and
include/gewell_b200_test.h (test and tuning aids) declare; layout helpers agree
with the oracle.  No compute call is made here."""
import re
from pathlib import Path

import numpy as np

from oracle import nvfp4 as onv

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols(header_name="gewell_b200.h"):
    header = (ROOT / "include" / header_name).read_text()
    return sorted(set(re.findall(r"\b(gw_[a-z0-9_]+)\s*\(", header)))


def test_library_exports_every_declared_symbol():
    from gewell_b200 import _lib
    lib = _lib.load()
    names = declared_symbols()
    aids = declared_symbols("gewell_b200_test.h")
    assert len(names) >= 40 and len(aids) >= 3
    assert not any(name.startswith("gw_debug_") and name != "gw_debug_kernel_error" for name in names), \
        "test aids belong in gewell_b200_test.h"
    for name in names + aids:
        assert hasattr(lib, name), f"{name} is declared in a header but not exported"
    assert set(names) | set(aids) == set(_lib.exported_symbols())
    assert lib.gw_abi_version() == 2


def test_layout_helpers_match_oracle():
    from gewell_b200 import _lib
    lib = _lib.load()
    for rows, width in [(1, 64), (128, 256), (129, 2816), (768, 2816), (5376, 21504)]:
        assert lib.gw_nvfp4_scale_storage_bytes(rows, width) == onv.scale_storage_bytes(rows, width)
    rng = np.random.default_rng(0)
    for _ in range(200):
        width = int(rng.integers(1, 100)) * 64
        row, block = int(rng.integers(0, 5000)), int(rng.integers(0, width // 16))
        assert lib.gw_nvfp4_scale_offset(row, block, width) == int(onv.scale_offset(row, block, width))
    # reference formulas: include/gewell/nvfp4_linear.h:42-49, fp8_linear.h:30-33
    assert lib.gw_nvfp4_scratch_upper_bound_bytes(33, 256, 256) == 64 * (128 + 512) + 2048 + 36 * 1024 * 1024 + 765
    assert lib.gw_fp8_scratch_upper_bound_bytes(33, 256) == 33 * 256 + 32 * 1024 * 1024 + 255


def test_no_gpu_calls_fail_cleanly_on_bad_arguments():
    """Argument validation happens before any CUDA call."""
    import ctypes
    from gewell_b200 import _lib
    lib = _lib.load()
    plan = ctypes.c_void_p()
    assert lib.gw_nvfp4_plan_create(0, 256, 256, ctypes.byref(plan)) == _lib.GW_INVALID_ARGUMENT
    assert b"K divisible by 64" in lib.gw_last_error()
    assert lib.gw_fp8_plan_create(1, 24, 16, 0, ctypes.byref(plan)) == _lib.GW_INVALID_ARGUMENT
    assert lib.gw_nvfp4_plan_create(4, 256, 256, ctypes.byref(plan)) == _lib.GW_OK
    assert lib.gw_nvfp4_plan_scratch_bytes(plan) == 512 + 2048
    lib.gw_nvfp4_plan_destroy(plan)
