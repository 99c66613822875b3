"""GPU tests of the BF16 plan and of the 26B projection binding / workspace
(bind_projection, ProjectionWorkspace: models/gemma4/26b_a4b/sm120/projection.cu:31-145)
through the C ABI.

The workspace test follows the design of the reference's own projection test
(tests/gemma4_26b_projection.cu:28-101): every weight row holds ONE non-zero
value, so each output is a single product that BF16 represents exactly; the
activations carry every E2M1 rounding tie, so the FP4-activation paths and the
BF16-activation paths have different, analytically known, results; padded
output rows of NVFP4 entries (704 -> 768) must never reach the caller; the
workspace's scratch must not grow."""
import struct

import numpy as np
import pytest
import torch

from oracle import codecs as C
from oracle import nvfp4 as onv
from tests.gpu_helpers import bf16_normal, bits, to_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gw():
    import gewell_b200
    return gewell_b200


@pytest.mark.parametrize("rows,k,n", [(1, 704, 2816), (7, 2816, 704), (64, 2816, 128), (128, 1024, 1408), (129, 2816, 704),
                                      (300, 704, 2816), (1024, 2816, 1408), (16, 5376, 8192)])
def test_bf16_plan_matches_fp32_matmul(gw, rows, k, n):
    """Y = bf16(X . W^T) with FP32 accumulation: against the FP64 dot, at the reference's own tolerance
    for its linear layers, max(0.8 % of |ref|, 1e-3).  Decode shapes run with and without the K split."""
    x = bf16_normal((rows, k), 11)
    w = bf16_normal((n, k), 12, 0.05)
    plan = gw.Bf16Plan(rows, k, n)
    expected = to_f32(x).astype(np.float64) @ to_f32(w).astype(np.float64).T
    results = []
    for with_scratch in (True, False):
        scratch = torch.full((plan.scratch_bytes() + 256,), 0xCD, dtype=torch.uint8, device="cuda") if with_scratch else None
        y = torch.full((rows * n + 64,), -3.0, dtype=torch.bfloat16, device="cuda")
        plan.run(x.cuda(), w.cuda(), y, scratch[:plan.scratch_bytes()] if with_scratch and plan.scratch_bytes() else None)
        torch.cuda.synchronize()
        assert gw.kernel_error() == 0
        assert torch.all(y[rows * n:] == -3.0), "wrote beyond the output"
        if with_scratch:
            assert torch.all(scratch[plan.scratch_bytes():] == 0xCD), "wrote beyond the scratch"
        got = to_f32(y[:rows * n].reshape(rows, n)).astype(np.float64)
        bound = np.maximum(0.008 * np.abs(expected), 0.001)
        assert np.isfinite(got).all() and (np.abs(got - expected) <= bound).all(), np.abs(got - expected).max()
        results.append(bits(y[:rows * n]))
    # BF16 products are exact in FP32 and so are most partial sums, but the K split changes the summation
    # order: the two runs agree to rounding, not necessarily bit for bit
    assert np.mean(results[0] != results[1]) < 0.02


def test_bf16_plan_validation(gw):
    with pytest.raises(gw.GewellInvalidArgument):
        gw.Bf16Plan(0, 64, 64)
    with pytest.raises(gw.GewellInvalidArgument):
        gw.Bf16Plan(1, 60, 64)
    with pytest.raises(gw.GewellInvalidArgument):
        gw.Bf16Plan(1, 64, 60)
    plan = gw.Bf16Plan(4, 64, 64)
    with pytest.raises(gw.GewellInvalidArgument):
        plan.run(None, None, None)


# ----------------------------------------------------------------------------- projection workspace

E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], dtype=np.float32)
RAW = np.array([0, .25, .75, 1.25, 1.75, 2.5, 3.5, 5, 6, -.25, -.75, -1.25, -1.75, -2.5, -3.5, -6], dtype=np.float32)
# nearest-even E2M1 value of every entry of RAW (ties go to the even code)
ROUNDED = np.array([0, 0, 1, 1, 2, 2, 4, 4, 6, 0, -1, -1, -2, -2, -4, -6], dtype=np.float32)


def activations(rows, k, fp4):
    """X[r, c]: a tie value of its K16 block position times the block's power-of-two scale."""
    r, c = np.meshgrid(np.arange(rows), np.arange(k), indexing="ij")
    block_scale = np.array([.5, 1., 2.], dtype=np.float32)[(c // 16 + r) % 3]
    values = (ROUNDED if fp4 else RAW)[c % 16] * np.float32(.125) * block_scale
    return np.where(r % 2 == 1, -values, values).astype(np.float32)


def row_code(n):
    return (1 + n % 7 + np.where(n % 2 == 1, 8, 0)).astype(np.uint8)


def coefficient(n):
    code = row_code(n)
    return E2M1[code & 7] * np.where(code & 8, -1.0, 1.0).astype(np.float32) * np.float32(.25)


def hot_column(n, k):
    return (n * 37 + 5) % k


def make_entry(storage, n, k):
    """Payload bytes of a one-hot [n, k] matrix in the given storage, artifact layout."""
    from gewell_b200 import _lib
    rows = np.arange(n)
    cols = hot_column(rows, k)
    if storage == _lib.STORAGE_BF16:
        w = np.zeros((n, k), dtype=np.float32)
        w[rows, cols] = coefficient(rows)
        return C.bf16_bits(w).tobytes()
    globals_ = struct.pack("<ff", 0.25, 0.125)          # weight_scale, input_scale
    if storage == _lib.STORAGE_FP8_W8A8:
        w = np.zeros((n, k), dtype=np.float32)
        w[rows, cols] = coefficient(rows) / np.float32(.25)
        return C.e4m3_encode(w).tobytes() + globals_
    physical = (n + 127) // 128 * 128
    codes = np.zeros((physical, k), dtype=np.uint8)
    codes[rows, cols] = row_code(rows)
    linear = np.zeros((physical, k // 16), dtype=np.uint8)
    linear[:n] = 0x38                                   # block scale 1.0; padding rows keep zero scales
    return C.pack_nibbles(codes).tobytes() + onv.tile_scales(linear, k).tobytes() + globals_


@pytest.mark.parametrize("n,k", [(704, 2816), (2112, 2816), (2816, 704), (2816, 2112), (4096, 2816), (1024, 2816),
                                 (2816, 4096)])
@pytest.mark.parametrize("storage_name", ["bf16", "fp8", "nvfp4"])
def test_projection_workspace_one_hot(gw, n, k, storage_name):
    from gewell_b200 import _lib
    storage = {"bf16": _lib.STORAGE_BF16, "fp8": _lib.STORAGE_FP8_W8A8, "nvfp4": _lib.STORAGE_NVFP4_W4A4}[storage_name]
    capacity = 160
    payload = make_entry(storage, n, k)
    device = torch.frombuffer(bytearray(payload), dtype=torch.uint8).cuda()
    projection = gw.bind_projection(storage, n, k, payload, device)
    physical = (n + 127) // 128 * 128 if storage == _lib.STORAGE_NVFP4_W4A4 else n
    assert (projection.input, projection.output, projection.physical_output) == (k, n, physical)
    if storage != _lib.STORAGE_BF16:
        scale = projection.nvfp4_weight_scale if storage == _lib.STORAGE_NVFP4_W4A4 else projection.fp8_weight_scale
        assert scale == 0.25
    x = torch.from_numpy(activations(capacity, k, False)).to(torch.bfloat16).cuda()
    coefficients = coefficient(np.arange(n))
    columns = hot_column(np.arange(n), k)
    stream = torch.cuda.current_stream()
    for policy in (_lib.POLICY_ALWAYS, _lib.POLICY_PREFILL):
        ws = gw.ProjectionWorkspace([projection], capacity, policy, stream)
        nbytes = ws.bytes()
        if storage == _lib.STORAGE_BF16:
            assert nbytes == 0, "BF16 projections need no scratch"
        for rows in (1, 33, 7, 129, capacity, 1):
            for phase in (_lib.PHASE_PREFILL, _lib.PHASE_DECODE):
                ws.prepare(rows, phase)
                y = torch.full((rows * n + 128,), -9.0, dtype=torch.bfloat16, device="cuda")
                ws.run(projection, x, y)
                torch.cuda.synchronize()
                assert gw.kernel_error() == 0
                fp4 = storage == _lib.STORAGE_NVFP4_W4A4 and gw.lib.gw_nvfp4_fp4_activations(policy, phase) != 0
                expected = C.bf16_round(activations(rows, k, fp4)[:, columns] * coefficients[None, :])
                got = to_f32(y[:rows * n].reshape(rows, n))
                # the sign of a zero is immaterial; every other BF16 value must be exact
                assert np.array_equal(got, expected), (storage_name, policy, phase, rows, np.abs(got - expected).max())
                assert torch.all(y[rows * n:] == -9.0), "projection wrote beyond its logical output"
                assert ws.bytes() == nbytes, "projection scratch grew during execution"


def test_projection_workspace_mixed_shapes_share_scratch(gw):
    """Several shapes and storage types behind one workspace (tests/gemma4_26b_projection.cu:103-157):
    constant weights, constant rows, so every output is K times one product."""
    from gewell_b200 import _lib
    cases = [(704, 2816, _lib.STORAGE_NVFP4_W4A4), (2112, 2816, _lib.STORAGE_FP8_W8A8), (2816, 704, _lib.STORAGE_NVFP4_W4A4),
             (2816, 2112, _lib.STORAGE_BF16)]
    keep, projections = [], []
    for n, k, storage in cases:
        if storage == _lib.STORAGE_BF16:
            payload = C.bf16_bits(np.full((n, k), 0.25, dtype=np.float32)).tobytes()
        elif storage == _lib.STORAGE_FP8_W8A8:
            payload = bytes([0x38]) * (n * k) + struct.pack("<ff", 0.25, 0.125)        # E4M3 1.0
        else:
            physical = (n + 127) // 128 * 128
            codes = np.zeros((physical, k // 2), dtype=np.uint8)
            codes[:n] = 0x22                                                          # E2M1 1.0 in both nibbles
            linear = np.zeros((physical, k // 16), dtype=np.uint8)
            linear[:n] = 0x38
            payload = codes.tobytes() + onv.tile_scales(linear, k).tobytes() + struct.pack("<ff", 0.25, 0.125)
        device = torch.frombuffer(bytearray(payload), dtype=torch.uint8).cuda()
        keep.append(device)
        projections.append(gw.bind_projection(storage, n, k, payload, device))
    for policy in (_lib.POLICY_ALWAYS, _lib.POLICY_PREFILL):
        ws = gw.ProjectionWorkspace(projections, 33, policy, torch.cuda.current_stream())
        nbytes = ws.bytes()
        for rows in (3, 33, 3):
            for phase in (_lib.PHASE_PREFILL, _lib.PHASE_DECODE):
                ws.prepare(rows, phase)
                for projection in projections:
                    values = np.where(np.arange(rows) % 2 == 1, 1.5, .75).astype(np.float32)
                    x = torch.from_numpy(np.repeat(values[:, None], projection.input, axis=1)).to(torch.bfloat16).cuda()
                    y = torch.full((rows * projection.output + 128,), -9.0, dtype=torch.bfloat16, device="cuda")
                    ws.run(projection, x, y)
                    torch.cuda.synchronize()
                    assert gw.kernel_error() == 0
                    expected = C.bf16_round((values * np.float32(.25) * projection.input).astype(np.float32))
                    got = to_f32(y[:rows * projection.output].reshape(rows, projection.output))
                    assert np.array_equal(got, np.repeat(expected[:, None], projection.output, axis=1))
                    assert torch.all(y[rows * projection.output:] == -9.0)
                    assert ws.bytes() == nbytes


def test_projection_binding_validation(gw):
    from gewell_b200 import _lib
    device = torch.zeros(64, dtype=torch.uint8, device="cuda")
    with pytest.raises(gw.GewellInvalidArgument):
        gw.bind_projection(7, 16, 64, bytes(64), device)                       # unknown storage
    with pytest.raises(gw.GewellInvalidArgument):
        gw.bind_projection(_lib.STORAGE_FP8_W8A8, 16, 64, bytes(64), device)   # entry too short for weights + globals
    with pytest.raises(gw.GewellInvalidArgument):
        gw.ProjectionWorkspace([], 0, _lib.POLICY_ALWAYS)
    ws = gw.ProjectionWorkspace([], 8, _lib.POLICY_ALWAYS)
    with pytest.raises(gw.GewellInvalidArgument):
        ws.prepare(9, _lib.PHASE_DECODE)
