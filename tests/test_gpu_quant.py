"""GPU parity of the element-wise kernels against the CPU oracle: weight
dequantise / pack / QDQ (bit-exact) and activation quantisation."""
import json

import numpy as np
import pytest
import torch

from oracle import codecs as C
from oracle import fp8 as ofp8
from oracle import nvfp4 as onv
from tests.gpu_helpers import bf16_normal, bits, device_weight_to_oracle, oracle_weight_to_device, to_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gw():
    import gewell_b200
    return gewell_b200


def test_dequantize_every_scale_code_and_nibble(gw):
    """tests/nvfp4_linear_test.cu:100-145: every E4M3 scale code 0..126 times
    every nibble, both 128-row tiles; input_scale has no effect."""
    k = n = 256
    rng = np.random.default_rng(0)
    packed = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    packed[:, :8] = np.arange(8, dtype=np.uint8) * 0x11 + np.arange(8, dtype=np.uint8)[::-1] * 0  # all nibbles appear
    packed[0, :16] = [(i | ((15 - i) << 4)) for i in range(16)]
    r, b = np.meshgrid(np.arange(n), np.arange(k // 16), indexing="ij")
    linear = ((r * 17 + b) % 127).astype(np.uint8)
    w = onv.Weight(packed, onv.tile_scales(linear, k), float("nan"), 0.0737, n, k)
    expected = onv.dequantize(w)
    dev = oracle_weight_to_device(w)
    out = torch.full((n * k + 128,), -1.0, dtype=torch.bfloat16, device="cuda")
    gw.nvfp4_dequantize(dev, k, n, out)
    torch.cuda.synchronize()
    assert np.array_equal(bits(out[:n * k]).reshape(n, k), expected)
    assert torch.all(out[n * k:] == -1.0)          # guard untouched


@pytest.mark.parametrize("shape,seed", [((2816, 2816), 0), ((256, 192 + 64), 5), ((704, 2816), 9)])
def test_pack_weights_bit_exact(gw, shape, seed):
    n, k = shape
    w = bf16_normal(shape, seed, 0.02)
    expected = onv.pack_weights(to_f32(w), 0.125)
    dev = gw.nvfp4_pack_weights(w.cuda(), 0.125)
    torch.cuda.synchronize()
    assert np.float32(dev.weight_scale) == np.float32(expected.weight_scale)
    assert np.array_equal(dev.data.cpu().numpy(), expected.data)
    assert np.array_equal(dev.scales.cpu().numpy(), expected.scales)
    # round trip through the device dequantiser == oracle dequantiser
    if n % 128 == 0:
        restored = gw.nvfp4_dequantize(dev, k, n)
        assert np.array_equal(bits(restored), onv.dequantize(expected))


def test_pack_weights_edge_blocks(gw):
    """Zero blocks (scale 1 = 0x38), tiny blocks (clamp 2^-9), ties and saturation."""
    values = np.zeros((128, 64), dtype=np.float32)
    values[0, :2] = [2688., -2688.]
    values[0, 16:32] = [0, -0., .25, .75, 1.25, 1.75, 2.5, 3.5, 5, -5, 6, -6, 6, -6, .5, -.5]
    values[0, 48] = 2.0 ** -16
    values[5] = np.linspace(-3, 3, 64)
    w = torch.from_numpy(C.bf16_round(values)).to(torch.bfloat16)
    expected = onv.pack_weights(to_f32(w), 0.125)
    dev = gw.nvfp4_pack_weights(w.cuda(), 0.125)
    assert np.array_equal(dev.data.cpu().numpy(), expected.data)
    assert np.array_equal(dev.scales.cpu().numpy(), expected.scales)
    assert list(onv.untile_scales(dev.scales.cpu().numpy(), 1, 64)[0]) == [126, 56, 56, 1]


def _check_quantized(gw, packed_dev, scales_dev, x_f32, input_scale, rows, k):
    """Exact comparison: the oracle evaluates the recipe's three approximate
    reciprocals with the hardware instruction (gw.rcp_approx), everything else
    on the CPU.  The spread against correctly rounded reciprocals is reported."""
    got_packed = packed_dev.cpu().numpy()
    got_scales = onv.untile_scales(scales_dev.cpu().numpy(), rows, k)
    exact = onv.quantize_activations(x_f32, input_scale, rcp_fn=gw.rcp_approx)
    assert np.array_equal(got_scales, exact.scales_linear)
    assert np.array_equal(got_packed, exact.packed[:rows])
    nominal = onv.quantize_activations(x_f32, input_scale)
    print(f"rows={rows} K={k}: bytes differing from the correctly-rounded-reciprocal model: "
          f"{np.mean(got_packed != nominal.packed[:rows]):.2e} (scales {np.mean(got_scales != nominal.scales_linear):.2e})")
    return got_packed, got_scales


def test_quantize_activations_vllm_fixtures(gw, golden_dir):
    """tests/nvfp4_linear_test.cu:147-205: frozen scaled_fp4_quant outputs, exact."""
    fixtures = json.loads((golden_dir / "reference_vectors.json").read_text())["vllm_scaled_fp4_quant"]["fixtures"]
    for f in fixtures:
        x = torch.tensor(f["input"] * 4, dtype=torch.float32).to(torch.bfloat16).reshape(1, 64).cuda()
        packed, scales = gw.nvfp4_quantize_activations(x, f["global"])
        torch.cuda.synchronize()
        linear = onv.untile_scales(scales.cpu().numpy(), 1, 64)
        assert list(packed.cpu().numpy()[0, :8]) == f["packed"]
        assert linear[0, 0] == f["scale"]
        # padding of the scale tile is rewritten with zeros
        assert scales.cpu().numpy().sum() == int(linear.sum())


@pytest.mark.parametrize("rows,k", [(16, 2816), (1, 64), (33, 256), (129, 704)])
def test_quantize_activations_matches_oracle(gw, rows, k):
    x = bf16_normal((rows, k), 1)
    x[0, :16] = 0                       # zero block -> scale 0, codes 0
    if k >= 64:
        x[0, 16:32] *= 1e-6             # underflowing scale
        x[0, 32:48] *= 1000             # saturating scale / FP4
    input_scale = float(to_f32(x).__abs__().max() / 2688) if rows > 1 else 0.0113
    packed, scales = gw.nvfp4_quantize_activations(x.cuda(), input_scale)
    torch.cuda.synchronize()
    _check_quantized(gw, packed, scales, to_f32(x), input_scale, rows, k)


def test_quantize_gelu_fused_equals_separate(gw):
    """tests/nvfp4_linear_test.cu:298-376: GeGLU fused into the quantiser is
    bit-identical to GeGLU followed by plain quantisation."""
    rows, k = 19, 704
    x = bf16_normal((rows, 2 * k), 3)
    fused_p, fused_s = gw.nvfp4_quantize_activations(x.cuda(), 0.02, gelu=True)
    act_dev = gw.geglu_bf16(to_f32(x[:, :k]), to_f32(x[:, k:]))
    act = torch.from_numpy(act_dev).to(torch.bfloat16)
    sep_p, sep_s = gw.nvfp4_quantize_activations(act.cuda(), 0.02)
    torch.cuda.synchronize()
    assert torch.equal(fused_p, sep_p) and torch.equal(fused_s, sep_s)
    # host tanh vs device tanhf: the two GeGLUs agree except for rare one-ulp BF16 flips
    host = C.gelu_tanh_multiply_bf16(to_f32(x[:, :k]), to_f32(x[:, k:]))
    assert np.mean(host != act_dev) < 5e-3
    assert np.max(np.abs(host - act_dev) / np.maximum(np.abs(host), 1e-30)) < 2 ** -6


def test_fp8_quantize_exact(gw):
    """tests/fp8_linear_test.cu:232-275: every RNE midpoint, subnormals,
    saturation at +-464 / +-FLT_MAX, several scales -- exact."""
    k = 256
    mags = C.E4M3_MAGNITUDES[:127]
    for scale in (1.0, 0.125, 0.0737, 8.0):
        vals = np.empty(k, dtype=np.float32)
        for i in range(k):
            code = (i // 2) % 126
            v = (mags[code] + mags[code + 1]) / 2
            vals[i] = (-v if i & 1 else v) * scale
        vals[:8] = [0.0, -0.0, 1 / 2048, 3 / 2048, 464.0, -464.0, np.finfo(np.float32).max, -np.finfo(np.float32).max]
        x = torch.from_numpy(vals).to(torch.bfloat16).reshape(1, k)
        got = gw.fp8_quantize_activations(x.cuda(), scale).cpu().numpy()
        with np.errstate(over="ignore"):
            expected = ofp8.quantize_activations(to_f32(x), scale)
        assert np.array_equal(got, expected), scale
    x = bf16_normal((37, 5376), 4)
    got = gw.fp8_quantize_activations(x.cuda(), 0.01).cpu().numpy()
    assert np.array_equal(got, ofp8.quantize_activations(to_f32(x), 0.01))
    # 2-byte aligned input takes the scalar path and gives the same bytes
    flat = torch.empty(37 * 5376 + 1, dtype=torch.bfloat16, device="cuda")
    flat[1:] = x.cuda().reshape(-1)
    got2 = gw.fp8_quantize_activations(flat[1:].view(37, 5376), 0.01).cpu().numpy()
    assert np.array_equal(got2, got)


def test_fp8_pack_weights(gw):
    w = bf16_normal((256, 512), 2, 0.02)
    exp_tensor = ofp8.pack_weights(to_f32(w))
    got = gw.fp8_pack_weights(w.cuda(), exp_tensor.weight_scale)
    assert np.array_equal(got.cpu().numpy(), exp_tensor.data)
    exp_rows = ofp8.pack_weights_per_channel(to_f32(w), 0.01)
    rs = torch.from_numpy(exp_rows.channel_weight_scales).cuda()
    got = gw.fp8_pack_weights(w.cuda(), 0.0, rs)
    assert np.array_equal(got.cpu().numpy(), exp_rows.data)


def test_qdq_goldens_on_device(gw, golden_dir):
    """tests/weight_qdq_test.cu:324-370 golden BF16 words through the device kernels."""
    v = json.loads((golden_dir / "reference_vectors.json").read_text())
    g = v["fp8_qdq"]
    inp = np.array([int(w, 16) for w in g["input_words"]], dtype=np.uint16)
    t = torch.from_numpy(inp.view(np.int16)).cuda().view(torch.bfloat16)
    gw.weight_qdq_apply(1, t)
    assert [f"{w:04x}" for w in bits(t)] == g["output_words"]
    g = v["nvfp4_qdq"]
    inp = np.zeros(g["length"], dtype=np.uint16)
    out = np.zeros(g["length"], dtype=np.uint16)
    for i, w in g["input_words"].items():
        inp[int(i)] = int(w, 16)
    for i, w in g["output_words"].items():
        out[int(i)] = int(w, 16)
    t = torch.from_numpy(inp.view(np.int16)).cuda().view(torch.bfloat16)
    gw.weight_qdq_apply(2, t)
    assert np.array_equal(bits(t), out)


@pytest.mark.parametrize("kind", [1, 2])
def test_qdq_matches_oracle_and_rejects_nonfinite(gw, kind):
    """tests/weight_qdq_test.cu:406-546: device == host bit-exact on a tensor
    larger than the capped grid; neighbours untouched; non-finite rejected."""
    n = 1_200_000 - (1_200_000 % 16)
    x = bf16_normal((n,), 6, 0.05)
    buf = torch.full((n + 64,), 7.0, dtype=torch.bfloat16, device="cuda")
    buf[32:32 + n] = x.cuda()
    gw.weight_qdq_apply(kind, buf[32:32 + n])
    expected = (ofp8.qdq if kind == 1 else onv.qdq)(bits(x))
    assert np.array_equal(bits(buf[32:32 + n]), expected)
    assert torch.all(buf[:32] == 7.0) and torch.all(buf[32 + n:] == 7.0)
    bad = x.clone().cuda()
    bad[12345] = float("inf")
    with pytest.raises(gw.GewellInvalidArgument):
        gw.weight_qdq_apply(kind, bad)
    zero = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    gw.weight_qdq_apply(kind, zero)
    assert torch.all(zero == 0)
