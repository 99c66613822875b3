"""GPU parity of the NVFP4 and FP8 linear layers (through the C ABI plans)
against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import codecs as C
from oracle import fp8 as ofp8
from oracle import nvfp4 as onv
from tests.gpu_helpers import (assert_gemm_close, assert_reference_tolerance, bf16_normal, bits,
                               oracle_weight_to_device, to_f32)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gw():
    import gewell_b200
    return gewell_b200


def run_nvfp4(gw, x, weight_dev, n, k, gelu=False, guard=True):
    rows = x.shape[0]
    plan = gw.Nvfp4Plan(rows, k, n)
    need = plan.scratch_bytes()
    assert need <= gw.lib.gw_nvfp4_scratch_upper_bound_bytes(rows, k, n)
    scratch = torch.full((need + 256,), 0xCD, dtype=torch.uint8, device="cuda")
    y = torch.full((rows * n + 128,), -7.0, dtype=torch.bfloat16, device="cuda")
    plan.run(x, weight_dev, y, scratch, need, transform=1 if gelu else 0)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    if guard:
        assert torch.all(scratch[need:] == 0xCD), "wrote beyond the scratch"
        assert torch.all(y[rows * n:] == -7.0), "wrote beyond the output"
    packed = scratch[:rows * k // 2].reshape(rows, k // 2).cpu().numpy()
    off = (rows * k // 2 + 255) // 256 * 256
    scales = scratch[off:off + onv.scale_storage_bytes(rows, k)].cpu().numpy()
    return y[:rows * n].reshape(rows, n), packed, scales


def oracle_from_device_quantisation(packed, scales, rows, k, weight):
    """FP64 dot over the activations exactly as the device quantised them:
    isolates the GEMM from the approximate-reciprocal uncertainty."""
    q = onv.QuantizedActivations(packed, onv.untile_scales(scales, rows, k), scales, rows, rows, k)
    return onv.linear_w4a4_from_quantized(onv.dequantized_activations(q), weight)


def test_config1_nvfp4_linear(gw):
    """W [2816,2816] ~ N(0,0.02) seed 0, X [16,2816] ~ N(0,1) seed 1."""
    n = k = 2816
    w = onv.pack_weights(to_f32(bf16_normal((n, k), 0, 0.02)))
    x = bf16_normal((16, k), 1)
    w.input_scale = float(np.abs(to_f32(x)).max() / 2688)
    y, packed, scales = run_nvfp4(gw, x.cuda(), oracle_weight_to_device(w), n, k)
    exact = oracle_from_device_quantisation(packed, scales, 16, k, w)
    assert_reference_tolerance(bits(y), exact, "config 1 vs FP64 dot of device-quantised operands")
    faithful = onv.linear_w4a4(to_f32(x), w, rcp_fn=gw.rcp_approx)
    m = assert_gemm_close(bits(y), faithful, "config 1 vs faithful W4A4 oracle")
    host_path = onv.linear_w4a16(to_f32(x), w)
    from tests.gpu_helpers import error_metrics
    print("config1 W4A4 oracle", m, "W4A16 host path", error_metrics(bits(y), host_path))


def test_scale_layout_with_distinct_powers_of_two(gw):
    """Every weight row and every K16 block carries its own power-of-two scale
    and the activations likewise; a wrong scale-tile mapping in the tensor
    core cannot produce the expected values."""
    n, k, rows = 256, 512, 48
    rng = np.random.default_rng(1)
    codes = rng.integers(1, 8, (n, k)).astype(np.uint8) | (rng.integers(0, 2, (n, k)).astype(np.uint8) << 3)
    r, b = np.meshgrid(np.arange(n), np.arange(k // 16), indexing="ij")
    linear = (0x38 + 8 * ((r * 5 + b * 3) % 7 - 3)).astype(np.uint8)       # 2^-3 .. 2^3
    w = onv.Weight(C.pack_nibbles(codes), onv.tile_scales(linear, k), 1.0, 1.0, n, k)
    xs = rng.integers(-6, 7, (rows, k)).astype(np.float32) * 0.5
    xs *= np.exp2(((np.arange(rows)[:, None] * 3 + (np.arange(k)[None, :] // 16)) % 5) - 2).astype(np.float32)
    x = torch.from_numpy(xs).to(torch.bfloat16)
    w.input_scale = 1.0 / 16
    y, packed, scales = run_nvfp4(gw, x.cuda(), oracle_weight_to_device(w), n, k)
    exact = oracle_from_device_quantisation(packed, scales, rows, k, w)
    assert_reference_tolerance(bits(y), exact, "power-of-two scale layout")


@pytest.mark.parametrize("k,n", [(256, 256), (64, 128), (704, 2816), (2816, 768)])
@pytest.mark.parametrize("rows", [1, 3, 17, 31, 32, 33, 127, 128, 129, 300])
def test_nvfp4_shapes(gw, k, n, rows):
    """Row counts around every tile boundary (tests/nvfp4_linear_test.cu:394-420),
    with zero, underflowing and saturating blocks in the input (:212-222)."""
    w = onv.pack_weights(to_f32(bf16_normal((n, k), 10 + n % 7, 0.05)), 0.0113)
    col = np.arange(k)
    vals = (((col[None, :] * 31 + np.arange(rows)[:, None] * 7 + col[None, :] // 13) % 127) - 63) / 8.0
    vals = vals.astype(np.float32)
    sel = (col // 16) % 17
    vals[:, sel == 0] = 0.0
    vals[:, sel == 1] *= 1e-6
    vals[:, sel == 2] *= 128
    x = torch.from_numpy(vals).to(torch.bfloat16)
    y, packed, scales = run_nvfp4(gw, x.cuda(), oracle_weight_to_device(w), n, k)
    exact = oracle_from_device_quantisation(packed, scales, rows, k, w)
    assert_reference_tolerance(bits(y), exact, f"rows={rows} K={k} N={n}")


@pytest.mark.parametrize("rows,k,n", [(640, 512, 8192), (520, 1024, 8192 + 128)])
def test_nvfp4_prefill_tiles_that_do_not_fill_whole_waves(gw, rows, k, n):
    """More 128x256 tiles than SMs but not a multiple of them (the last wave is ragged), wide N,
    two launches on one plan must agree bit for bit."""
    w = onv.pack_weights(to_f32(bf16_normal((n, k), 21, 0.05)), 0.0113)
    x = bf16_normal((rows, k), 22)
    dev = oracle_weight_to_device(w)
    plan = gw.Nvfp4Plan(rows, k, n)
    scratch = torch.empty(plan.scratch_bytes(), dtype=torch.uint8, device="cuda")
    assert plan.scratch_bytes() <= gw.lib.gw_nvfp4_scratch_upper_bound_bytes(rows, k, n)
    y = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    results = []
    for _ in range(2):
        y.fill_(float("nan"))
        plan.run(x.cuda(), dev, y, scratch)
        torch.cuda.synchronize()
        assert gw.kernel_error() == 0
        results.append(bits(y).copy())
    assert np.array_equal(results[0], results[1])
    packed = scratch[:rows * k // 2].cpu().numpy().reshape(rows, k // 2)
    scales = scratch[(rows * k // 2 + 255) // 256 * 256:][:onv.scale_storage_bytes(rows, k)].cpu().numpy()
    exact = oracle_from_device_quantisation(packed, scales, rows, k, w)
    assert_reference_tolerance(results[0], exact, f"prefill rows={rows} K={k} N={n}")


@pytest.mark.parametrize("k,n", [(192, 256), (1344, 640), (2816, 384)])
@pytest.mark.parametrize("rows", [256, 257, 385, 512, 1000])
def test_nvfp4_cta_pair_tile_edges(gw, k, n, rows, monkeypatch):
    """From 256 rows the projection runs on CTA pairs (256-token x 256-channel tiles).  Row counts
    that leave the second CTA of a pair empty, partly filled or full; K with a partial last stage
    and K longer than the stage ring; channel counts with a ragged last tile.  The single-CTA
    kernel must give the same bits on the same quantised input."""
    w = onv.pack_weights(to_f32(bf16_normal((n, k), 31 + n % 5, 0.05)), 0.0113)
    dev = oracle_weight_to_device(w)
    x = bf16_normal((rows, k), 32 + rows % 11).cuda()
    y_pair, packed, scales = run_nvfp4(gw, x, dev, n, k)
    exact = oracle_from_device_quantisation(packed, scales, rows, k, w)
    assert_reference_tolerance(bits(y_pair), exact, f"pair rows={rows} K={k} N={n}")
    monkeypatch.setenv("GW_DENSE_NO_PAIR", "1")
    y_single, _, _ = run_nvfp4(gw, x, dev, n, k)
    assert np.array_equal(bits(y_pair), bits(y_single))


@pytest.mark.parametrize("form", ["direct", "swap"])
@pytest.mark.parametrize("rows", [5, 64, 128])
def test_nvfp4_both_operand_roles(gw, form, rows, monkeypatch):
    """Small row counts normally put the weights on the lane operand; the other
    role assignment must give the same numbers."""
    monkeypatch.setenv("GW_DENSE_FORM", form)
    n, k = 384, 704
    w = onv.pack_weights(to_f32(bf16_normal((n, k), 8, 0.05)), 0.0113)
    x = bf16_normal((rows, k), 9)
    y, packed, scales = run_nvfp4(gw, x.cuda(), oracle_weight_to_device(w), n, k)
    exact = oracle_from_device_quantisation(packed, scales, rows, k, w)
    assert_reference_tolerance(bits(y), exact, f"{form} rows={rows}")


def test_nvfp4_gelu_input(gw):
    n, k, rows = 256, 704, 21
    w = onv.pack_weights(to_f32(bf16_normal((n, k), 3, 0.05)), 0.02)
    x = bf16_normal((rows, 2 * k), 4)
    y, packed, scales = run_nvfp4(gw, x.cuda(), oracle_weight_to_device(w), n, k, gelu=True)
    exact = oracle_from_device_quantisation(packed, scales, rows, k, w)
    assert_reference_tolerance(bits(y), exact, "GeGLU input")
    faithful = onv.linear_w4a4(to_f32(x), w, gelu=True, rcp_fn=gw.rcp_approx, gelu_fn=gw.geglu_bf16)
    assert_gemm_close(bits(y), faithful, "GeGLU input vs faithful oracle")


def test_nvfp4_argument_validation(gw):
    """tests/nvfp4_linear_test.cu:421-423 and src/nvfp4_linear.cu:157-164,278-288."""
    for bad in [(0, 256, 256), (1, 0, 256), (1, 250, 256), (1, 256, 0), (1, 256, 200)]:
        with pytest.raises(gw.GewellInvalidArgument):
            gw.Nvfp4Plan(*bad)
    plan = gw.Nvfp4Plan(4, 256, 256)
    w = oracle_weight_to_device(onv.pack_weights(to_f32(bf16_normal((256, 256), 1, 0.05)), 0.01))
    x = bf16_normal((4, 256), 2).cuda()
    y = torch.empty((4, 256), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(plan.scratch_bytes() + 512, dtype=torch.uint8, device="cuda")
    with pytest.raises(gw.GewellInvalidArgument):
        plan.run(x, w, y, scratch, plan.scratch_bytes() - 1)
    with pytest.raises(gw.GewellInvalidArgument):
        plan.run(x, w, y, scratch[1:], plan.scratch_bytes())
    for scale in (0.0, -1.0, float("nan"), float("inf"), 1e-45):
        with pytest.raises(gw.GewellInvalidArgument):
            plan.run(x, gw.Nvfp4Weight(w.data, w.scales, scale, w.weight_scale), y, scratch, plan.scratch_bytes())
    with pytest.raises(gw.GewellInvalidArgument):
        plan.run(x, w, y, scratch, plan.scratch_bytes(), transform=5)
    with pytest.raises(gw.GewellInvalidArgument):
        gw.nvfp4_dequantize(w, 250, 256)


def test_w4a16_projection(gw):
    """BF16 activations x NVFP4 weights for 1..8 rows vs the host path
    (dequantise, FP32 matmul)."""
    n = k = 2816
    w = onv.pack_weights(to_f32(bf16_normal((n, k), 0, 0.02)))
    dev = oracle_weight_to_device(w)
    for rows in (1, 4, 8):
        x = bf16_normal((rows, k), 20 + rows)
        y = gw.nvfp4_gemv_w4a16(x.cuda(), dev, k, n)
        torch.cuda.synchronize()
        assert_gemm_close(bits(y), onv.linear_w4a16(to_f32(x), w), f"W4A16 rows={rows}")


# --------------------------------------------------------------------------- FP8

def run_fp8(gw, x, weight, n, k, channel=False, gelu=False):
    rows = x.shape[0]
    plan = gw.Fp8Plan(rows, k, n, channel)
    need = plan.scratch_bytes()
    assert need <= gw.lib.gw_fp8_scratch_upper_bound_bytes(rows, k)
    scratch = torch.full((need + 256,), 0xCD, dtype=torch.uint8, device="cuda")
    y = torch.full((rows * n + 128,), -7.0, dtype=torch.bfloat16, device="cuda")
    plan.run(x, weight, y, scratch, need, transform=1 if gelu else 0)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert torch.all(scratch[need:] == 0xCD) and torch.all(y[rows * n:] == -7.0)
    return y[:rows * n].reshape(rows, n)


def fp8_weight_to_device(gw, w: ofp8.Weight):
    cs = torch.from_numpy(w.channel_scales).cuda() if w.channel_scales is not None else None
    return gw.Fp8Weight(torch.from_numpy(w.data.copy()).cuda(), w.input_scale, w.weight_scale, cs)


@pytest.mark.parametrize("rows", [1, 8, 32, 64])
def test_config2_fp8_decode_slice(gw, rows):
    """Config 2 shapes (K=5376, per-output-channel scales) on a 4096-channel
    slice of the 43008 so that the FP64 oracle stays fast; the full width is
    covered by the property test below."""
    n, k = 4096, 5376
    wv = to_f32(bf16_normal((n, k), 2, 0.02))
    x = bf16_normal((rows, k), 30 + rows)
    input_scale = float(np.abs(to_f32(x)).max() / 448)
    w = ofp8.pack_weights_per_channel(wv, input_scale)
    y = run_fp8(gw, x.cuda(), fp8_weight_to_device(gw, w), n, k, channel=True)
    expected = ofp8.linear_w8a8(to_f32(x), w)
    assert_reference_tolerance(bits(y), expected, f"FP8 joined rows={rows}")
    from tests.gpu_helpers import error_metrics
    print("FP8 rows", rows, "vs W8A16 host path", error_metrics(bits(y), ofp8.linear_w8a16(to_f32(x), w)))


def test_fp8_rounding_boundaries_exact(gw):
    """tests/fp8_linear_test.cu:232-275: identity weights make the activation
    codes visible in the output; every signed weight code; zero input -- exact."""
    k = n = 256
    data = np.zeros((n, k), dtype=np.uint8)
    data[np.arange(n), np.arange(n)] = 0x38
    mags = C.E4M3_MAGNITUDES[:127]
    for scale in (1.0, 0.125, 0.0737, 8.0):
        vals = np.empty(k, dtype=np.float32)
        for i in range(k):
            code = (i // 2) % 126
            v = (mags[code] + mags[code + 1]) / 2
            vals[i] = (-v if i & 1 else v) * scale
        vals[:8] = [0.0, -0.0, 1 / 2048, 3 / 2048, 464.0, -464.0, np.finfo(np.float32).max, -np.finfo(np.float32).max]
        x = torch.from_numpy(vals).to(torch.bfloat16).reshape(1, k)
        w = ofp8.Weight(data, scale, 0.25)
        y = run_fp8(gw, x.cuda(), fp8_weight_to_device(gw, w), n, k)
        with np.errstate(over="ignore"):
            assert np.array_equal(bits(y), ofp8.linear_w8a8(to_f32(x), w)), scale
    data = np.zeros((n, k), dtype=np.uint8)
    data[:, 0] = [(r % 127) | ((r // 127) % 2 * 128) for r in range(n)]
    x = torch.zeros((1, k), dtype=torch.bfloat16)
    x[0, 0] = 1
    w = ofp8.Weight(data, 1.0, 0.0737)
    y = run_fp8(gw, x.cuda(), fp8_weight_to_device(gw, w), n, k)
    assert np.array_equal(bits(y), ofp8.linear_w8a8(to_f32(x), w))
    y = run_fp8(gw, torch.zeros((1, k), dtype=torch.bfloat16, device="cuda"),
                fp8_weight_to_device(gw, ofp8.Weight(data, 0.0113, 0.0737)), n, k)
    assert torch.all(y == 0)


@pytest.mark.parametrize("rows", [1, 2, 3, 4])
@pytest.mark.parametrize("channel", [False, True])
def test_fp8_cuda_core_weight_streaming(gw, rows, channel, monkeypatch):
    """The optional CUDA-core decode path (GW_FP8_GEMV_ROWS) quantises the activations itself
    and must agree with the W8A8 oracle like the tensor-core path."""
    monkeypatch.setenv("GW_FP8_GEMV_ROWS", "4")
    n, k = 640, 5376
    wv = to_f32(bf16_normal((n, k), 43, 0.05))
    x = bf16_normal((rows, k), 44)
    w = ofp8.pack_weights_per_channel(wv, 0.02) if channel else ofp8.pack_weights(wv, 0.02)
    y = run_fp8(gw, x.cuda(), fp8_weight_to_device(gw, w), n, k, channel=channel)
    assert_reference_tolerance(bits(y), ofp8.linear_w8a8(to_f32(x), w), f"FP8 CUDA-core rows={rows}")


@pytest.mark.parametrize("k,n", [(16, 16), (256, 272), (5376, 512)])
@pytest.mark.parametrize("rows", [1, 2, 3, 15, 17, 33, 65, 129, 257])
def test_fp8_shapes(gw, k, n, rows):
    wv = to_f32(bf16_normal((n, k), 40, 0.05))
    x = bf16_normal((rows, k), 41)
    w = ofp8.pack_weights(wv, 0.02)
    y = run_fp8(gw, x.cuda(), fp8_weight_to_device(gw, w), n, k)
    assert_reference_tolerance(bits(y), ofp8.linear_w8a8(to_f32(x), w), f"FP8 rows={rows} K={k} N={n}")


def test_fp8_gelu_and_validation(gw):
    n, k, rows = 256, 512, 9
    w = ofp8.pack_weights(to_f32(bf16_normal((n, k), 50, 0.05)), 0.02)
    x = bf16_normal((rows, 2 * k), 51)
    y = run_fp8(gw, x.cuda(), fp8_weight_to_device(gw, w), n, k, gelu=True)
    assert_gemm_close(bits(y), ofp8.linear_w8a8(to_f32(x), w, gelu=True), "FP8 GeGLU")
    for bad in [(0, 16, 16), (1, 0, 16), (1, 24, 16), (1, 16, 0), (1, 16, 24)]:
        with pytest.raises(gw.GewellInvalidArgument):
            gw.Fp8Plan(*bad)
    plan = gw.Fp8Plan(rows, k, n, True)
    dev = fp8_weight_to_device(gw, w)
    scratch = torch.empty(plan.scratch_bytes(), dtype=torch.uint8, device="cuda")
    yy = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(gw.GewellInvalidArgument):          # joined plan without channel scales
        plan.run(x[:, :k].contiguous().cuda(), dev, yy, scratch)
    with pytest.raises(gw.GewellInvalidArgument):
        gw.Fp8Plan(rows, k, n).run(x[:, :k].contiguous().cuda(), gw.Fp8Weight(dev.data, float("nan"), 1.0), yy, scratch)


def test_config2_full_width_property(gw):
    """Full config-2 size (N=43008): linearity in the per-channel scale and
    agreement of identical channel blocks -- size-independent checks where the
    FP64 oracle would take minutes."""
    n, k, rows = 43008, 5376, 8
    base = bf16_normal((512, k), 2, 0.02)
    wv = base.repeat(n // 512, 1)                         # 84 identical blocks of 512 channels
    scale_rows = torch.full((n,), 0.02 / 448, dtype=torch.float32)
    data = gw.fp8_pack_weights(wv.cuda(), 0.0, scale_rows.cuda())
    x = bf16_normal((rows, k), 33).cuda()
    cs1 = torch.full((n,), 1e-4, dtype=torch.float32, device="cuda")
    y1 = run_fp8(gw, x, gw.Fp8Weight(data, 0.01, 1.0, cs1), n, k, channel=True)
    y2 = run_fp8(gw, x, gw.Fp8Weight(data, 0.01, 1.0, cs1 * 2), n, k, channel=True)
    assert torch.equal(y2.float(), y1.float() * 2)        # power-of-two scale: exact
    blocks = y1.reshape(rows, n // 512, 512)
    assert torch.equal(blocks, blocks[:, :1].expand_as(blocks))
    small = ofp8.Weight(data[:512].cpu().numpy(), 0.01, 1.0, np.full(512, 1e-4, np.float32))
    assert_reference_tolerance(bits(y1[:, :512]), ofp8.linear_w8a8(to_f32(x), small), "first block vs oracle")
