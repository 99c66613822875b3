"""GPU parity of the MoE layer (routing, permutation, grouped expert GEMMs,
GeGLU, ordered combine) against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest
import torch

from oracle import codecs as C
from oracle import moe as omoe
from oracle import nvfp4 as onv
from tests.gpu_helpers import assert_gemm_close, bf16_normal, bits, error_metrics, to_f32

pytestmark = pytest.mark.gpu

E, H, I = 128, 2816, 704


@pytest.fixture(scope="module")
def gw():
    import gewell_b200
    return gewell_b200


def pack_padded(gw, w_bf16, input_scale, physical_rows):
    """Device-pack [rows,K] and place it in a zero buffer of `physical_rows`
    rows (the 26B artifact pads N to 128 with zero rows and zero scales)."""
    rows, k = w_bf16.shape
    packed = gw.nvfp4_pack_weights(w_bf16, input_scale)
    if physical_rows != rows:
        data = torch.zeros((physical_rows, k // 2), dtype=torch.uint8, device=w_bf16.device)
        data[:rows] = packed.data
        packed = gw.Nvfp4Weight(data, packed.scales, packed.input_scale, packed.weight_scale)
    return packed


@pytest.fixture(scope="module")
def experts(gw):
    """128 experts, gate/up [704,2816] and down [2816,704] ~ N(0,0.02) from
    seed 4 with per-expert sub-seeds; packed on the device (that packer is
    checked bit-exact against the oracle in test_gpu_quant.py)."""
    device, host = [], []
    for e in range(E):
        g = torch.Generator().manual_seed(4 * 1000 + e)
        mats = [(torch.randn((I, H), generator=g) * 0.02).bfloat16(),
                (torch.randn((I, H), generator=g) * 0.02).bfloat16(),
                (torch.randn((H, I), generator=g) * 0.02).bfloat16()]
        scales = [0.004 + 0.0001 * (e % 5), 0.004 + 0.0001 * (e % 5) if e % 2 == 0 else 0.0045, 0.0007 + 0.00001 * (e % 3)]
        packs = [pack_padded(gw, m.cuda(), s, (m.shape[0] + 127) // 128 * 128) for m, s in zip(mats, scales)]
        device.append(tuple(packs))
        host.append(omoe.ExpertWeights(*[
            onv.Weight(p.data.cpu().numpy(), p.scales.cpu().numpy(), p.input_scale, p.weight_scale,
                       p.data.shape[0], m.shape[1]) for p, m in zip(packs, mats)]))
    return gw.ExpertTable(device), host


@pytest.fixture(scope="module")
def experts_shared(gw, experts):
    """The same matrices with one input scale for gate and up per expert (they
    are one fused tensor in the checkpoint): enables the fused GeGLU epilogue."""
    table, host = experts
    device = []
    shared_host = []
    for (gate, up, down), h in zip(table._keep, host):
        up2 = gw.Nvfp4Weight(up.data, up.scales, gate.input_scale, up.weight_scale)
        device.append((gate, up2, down))
        hu = onv.Weight(h.up.data, h.up.scales, h.gate.input_scale, h.up.weight_scale, h.up.rows, h.up.width)
        shared_host.append(omoe.ExpertWeights(h.gate, hu, h.down))
    return gw.ExpertTable(device), shared_host


@pytest.fixture
def moe_form():
    """Sets / clears the tuning overrides that select the grouped-GEMM plan (read when a workspace is
    created): "swap", "direct" or "fused", optionally followed by "-single" to keep the CTA-pair
    kernels out (the fused and direct plans then run on the single-CTA kernel)."""
    def choose(name):
        os.environ.pop("GW_MOE_FORM", None)
        os.environ.pop("GW_MOE_NO_PAIR", None)
        if name is not None:
            form, _, variant = name.partition("-")
            os.environ["GW_MOE_FORM"] = form
            if variant == "single":
                os.environ["GW_MOE_NO_PAIR"] = "1"
    yield choose
    os.environ.pop("GW_MOE_FORM", None)
    os.environ.pop("GW_MOE_NO_PAIR", None)


def make_scores(rows, mode, seed=0):
    if mode == "normal":
        return bf16_normal((rows, E), 100 + seed)
    scores = torch.full((rows, E), -4.0, dtype=torch.bfloat16)
    r = torch.arange(rows)
    starts = (r * 13) % E if mode == "distributed" else torch.where(r % 11 == 0, 120, 0) if mode == "uneven" else torch.zeros_like(r)
    ranks = torch.arange(8)
    scores.scatter_(1, (starts[:, None] + ranks) % E, (5.0 - ranks * .125).bfloat16().expand(rows, 8))
    if mode == "ties":
        scores.zero_()
    return scores


@pytest.mark.parametrize("rows,mode,launches", [
    (1, "hot", 1), (17, "distributed", 1), (65, "normal", 1), (129, "uneven", 1), (257, "distributed", 1), (17, "ties", 1),
    (4096, "hot", 1), (4096, "distributed", 1), (1000, "normal", 1), (8192, "normal", 1),
    # more chunks than resident blocks: several chunks per block of the one-launch kernel
    (40000, "normal", 1), (65536, "uneven", 1),
    (1000, "normal", 3), (8192, "normal", 3)])
def test_dispatch_exact(gw, rows, mode, launches, monkeypatch):
    """Selected ids, stable permutation and offsets are bit-exact; the FP32
    routing weights agree to a few ulps (host exp vs device expf).  From 65 tokens on
    routing, scan and scatter are one launch with a grid-wide barrier (or, on request,
    three launches)."""
    if launches == 3:
        monkeypatch.setenv("GW_MOE_ROUTE_THREE_LAUNCHES", "1")
    scores = make_scores(rows, mode)
    scales = C.bf16_round(1.0 + 0.1 * np.sin(np.arange(E, dtype=np.float32)))
    ws = gw.MoeWorkspace(rows)
    ws.dispatch(scores.cuda(), torch.from_numpy(scales).to(torch.bfloat16).cuda(), rows)
    torch.cuda.synchronize()
    ids, weights = omoe.route(to_f32(scores), scales)
    order, offsets = omoe.permutation(ids)
    assert np.array_equal(ws.selected_experts().cpu().numpy(), ids)
    np.testing.assert_allclose(ws.routing_weights().cpu().numpy(), weights, rtol=3e-6, atol=0)
    assert np.array_equal(ws.offsets().cpu().numpy(), offsets)
    assert np.array_equal(ws.sorted_assignments().cpu().numpy(), order)
    # run-to-run determinism (tests/gemma4_26b_moe.cu:74-77)
    first = ws.routing_weights().clone()
    ws.dispatch(scores.cuda(), torch.from_numpy(scales).to(torch.bfloat16).cuda(), rows)
    assert torch.equal(first, ws.routing_weights())


def test_dispatch_zero_rows_and_capacity(gw):
    ws = gw.MoeWorkspace(8)
    ws.dispatch(None, None, 0)                     # no-op (moe.cu:479)
    with pytest.raises(gw.GewellInvalidArgument):
        ws.dispatch(torch.zeros((9, E), dtype=torch.bfloat16, device="cuda"),
                    torch.ones(E, dtype=torch.bfloat16, device="cuda"), 9)
    with pytest.raises(gw.GewellInvalidArgument):
        gw.MoeWorkspace(0)


@pytest.mark.parametrize("width", [H, 704])
def test_combine_kernel_exact(gw, width):
    """Ordered BF16 fold, bit for bit: the layer's own width runs the block-per-token kernel with
    packed BF16 adds, any other width the generic kernel."""
    H = width
    rows = 37
    rng = np.random.default_rng(0)
    down = bf16_normal((rows * 8, H), 7)
    down[5, :8] = torch.tensor([0.0, -0.0, 1e-30, -1e-30, 3.0e38, -3.0e38, 1.0, -1.0], dtype=torch.bfloat16)
    weights = rng.random((rows, 8)).astype(np.float32)
    inverse = rng.permutation(rows * 8).astype(np.int32)
    out = gw.moe_combine(down.cuda(), torch.from_numpy(inverse).cuda(), torch.from_numpy(weights).cuda(), rows)
    torch.cuda.synchronize()
    assert np.array_equal(bits(out), omoe.combine(to_f32(down), inverse, weights))


@pytest.mark.parametrize("rows,mode,form", [
    (1, "hot", None), (7, "normal", None), (17, "distributed", None), (33, "normal", None), (64, "normal", None),
    (129, "uneven", None), (300, "normal", None),
    # an expert with 33..64 rows and a 32-row column tile: the second tile starts 32 rows into
    # its scale atom; 200 hot tokens walk a 64-row tile through all of an atom's offsets
    (40, "hot", None), (64, "hot", None), (200, "hot", None),
    (7, "normal", "direct"), (129, "uneven", "direct"), (300, "normal", "direct"),
    (1, "hot", "fused"), (33, "normal", "fused"), (129, "uneven", "fused"), (300, "normal", "fused"),
    # 200 hot tokens: eight experts with 200 rows each (a pair tile whose second CTA is partly filled);
    # 4096 uneven: experts with thousands of rows next to empty ones
    (200, "hot", "fused"), (600, "uneven", "fused"),
    (7, "normal", "direct-single"), (300, "normal", "direct-single"),
    (1, "hot", "fused-single"), (129, "uneven", "fused-single"), (300, "normal", "fused-single"),
])
def test_moe_layer_vs_oracle(gw, experts, experts_shared, moe_form, rows, mode, form):
    """Whole layer against the faithful W4A4 oracle, for each grouped-GEMM plan:
    swap (small batches), direct (tokens on the lane operand) and fused (GeGLU +
    quantisation in the gate/up epilogue; needs one input scale for gate and up).
    Fused and direct run their GEMMs on CTA pairs (gate/up only when fused; down in
    both) unless "-single" keeps them on the single-CTA kernel."""
    table, host = experts_shared if form is not None and form.startswith("fused") else experts
    moe_form(form)
    x = bf16_normal((rows, H), 200 + rows)
    scores = make_scores(rows, mode, rows)
    scales = np.ones(E, dtype=np.float32)
    ws = gw.MoeWorkspace(max(rows, 64))
    ws.capture(True)
    y = torch.full((rows * H + 64,), -3.0, dtype=torch.bfloat16, device="cuda")
    ws.run(x.cuda(), scores.cuda(), torch.ones(E, dtype=torch.bfloat16, device="cuda"), table, y, rows)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert torch.all(y[rows * H:] == -3.0)
    capture = {}
    expected = omoe.forward(to_f32(x), to_f32(scores), scales, host, capture=capture, rcp_fn=gw.rcp_approx,
                            gelu_fn=gw.geglu_bf16)
    assert np.array_equal(ws.selected_experts().cpu().numpy(), capture["ids"])
    assert np.array_equal(ws.sorted_assignments().cpu().numpy(), capture["order"])
    m_gu = assert_gemm_close(bits(ws.gate_up_capture()), C.bf16_bits(capture["gate_up"]), "gate/up capture")
    m_act = assert_gemm_close(bits(ws.activated_capture()), C.bf16_bits(capture["activated"]), "activated capture")
    m_dn = assert_gemm_close(bits(ws.down_capture()), C.bf16_bits(capture["down"]), "down capture")
    m = assert_gemm_close(bits(y[:rows * H].reshape(rows, H)), expected, f"MoE rows={rows} {mode} {form}")
    host_path = omoe.forward(to_f32(x), to_f32(scores), scales, host, mode="w4a16")
    print(f"rows={rows} {mode} {form}: gate_up {m_gu['rel_fro']:.2e} act {m_act['rel_fro']:.2e} down {m_dn['rel_fro']:.2e} "
          f"out {m['rel_fro']:.2e} max_abs/max {m['max_abs'] / m['max_ref']:.2e}; vs W4A16 host path "
          f"rel_fro {error_metrics(bits(y[:rows * H].reshape(rows, H)), host_path)['rel_fro']:.3f}")


def test_moe_fused_without_capture_matches_captured_run(gw, experts_shared, moe_form):
    """The fused plan skips the BF16 intermediates unless capture is on; the
    layer output must not depend on that switch."""
    table, _ = experts_shared
    moe_form("fused")
    rows = 257
    x = bf16_normal((rows, H), 91).cuda()
    scores = make_scores(rows, "normal", 9).cuda()
    one = torch.ones(E, dtype=torch.bfloat16, device="cuda")
    outs = []
    for capture in (False, True):
        ws = gw.MoeWorkspace(rows)
        ws.capture(capture)
        y = torch.empty((rows, H), dtype=torch.bfloat16, device="cuda")
        ws.run(x, scores, one, table, y, rows)
        torch.cuda.synchronize()
        outs.append(y)
    assert gw.kernel_error() == 0
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("rows,form", [(2048, None), (2048, "fused"), (8192, "fused"), (8192, "direct"),
                                       (2048, "fused-single"), (8192, "direct-single")])
def test_moe_layer_combine_consistency(gw, experts, experts_shared, moe_form, rows, form):
    """Size-independent properties at sizes where the full oracle is slow: the
    layer output is exactly the ordered BF16 fold of its own down capture
    (moe.cu:446-456), offsets are the histogram of the selected ids, and the
    plans agree with each other to GEMM tolerance."""
    table, _ = experts_shared if form is not None and form.startswith("fused") else experts
    moe_form(form)
    x = bf16_normal((rows, H), 77)
    scores = make_scores(rows, "normal", 5)
    ws = gw.MoeWorkspace(rows)
    y = torch.empty((rows, H), dtype=torch.bfloat16, device="cuda")
    ws.run(x.cuda(), scores.cuda(), torch.ones(E, dtype=torch.bfloat16, device="cuda"), table, y, rows)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    order = ws.sorted_assignments().cpu().numpy()
    inverse = np.empty_like(order)
    inverse[order] = np.arange(order.size, dtype=order.dtype)
    expected = omoe.combine(to_f32(ws.down_capture()), inverse, ws.routing_weights().cpu().numpy())
    assert np.array_equal(bits(y), expected)
    offsets = ws.offsets().cpu().numpy()
    ids = ws.selected_experts().cpu().numpy()
    assert offsets[-1] == rows * 8 and np.array_equal(np.bincount(ids.reshape(-1), minlength=E), np.diff(offsets))
    if form is not None:
        # same inputs through the small-batch plan: identical quantised operands, so the
        # two results differ only by FP32 accumulation order inside the tensor core
        moe_form("swap")
        ws2 = gw.MoeWorkspace(rows)
        y2 = torch.empty((rows, H), dtype=torch.bfloat16, device="cuda")
        ws2.run(x.cuda(), scores.cuda(), torch.ones(E, dtype=torch.bfloat16, device="cuda"), table, y2, rows)
        torch.cuda.synchronize()
        assert_gemm_close(bits(y), bits(y2), f"{form} plan vs swap plan at rows={rows}")


def test_moe_mode_validation(gw, experts):
    table, _ = experts
    ws = gw.MoeWorkspace(4)
    x = torch.zeros((4, H), dtype=torch.bfloat16, device="cuda")
    s = torch.zeros((4, E), dtype=torch.bfloat16, device="cuda")
    one = torch.ones(E, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(gw.GewellUnsupported, match="enable_w4a16"):
        ws.run(x, s, one, table, x.clone(), 4, fp4=False)          # W4A16 needs the BF16 copies first
    with pytest.raises(gw.GewellInvalidArgument):
        ws.run(x, s, one, table, x.clone(), 4, has_nvfp4=False)    # nothing selected
    ws.run(x, s, one, table, x.clone(), 4, has_bf16=True)          # extra flags are hints only
    ws.run(x, s, one, table, x.clone(), 0)                         # rows == 0 is a no-op
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0


@pytest.fixture(scope="module")
def experts_w4a16(gw, experts):
    """The NVFP4 experts with their BF16 copies made (a table of its own: the copies cost 1.6 GB)."""
    table, host = experts
    w4a16 = gw.ExpertTable(table._keep)
    w4a16.enable_w4a16()
    return w4a16, host


@pytest.mark.parametrize("rows,mode", [(1, "hot"), (7, "normal"), (33, "normal"), (129, "uneven"), (600, "uneven")])
def test_moe_w4a16_experts_vs_host_path(gw, experts_w4a16, rows, mode):
    """NVFP4 experts with BF16 activations (fp4 = 0; the reference's grouped_linear, moe.cu:96-103,353-395):
    against the W4A16 host path -- dequantise the weights to BF16, FP32 matmul -- at the path's tolerance."""
    table, host = experts_w4a16
    x = bf16_normal((rows, H), 400 + rows)
    scores = make_scores(rows, mode, rows)
    ws = gw.MoeWorkspace(max(rows, 64))
    y = torch.full((rows * H + 64,), -3.0, dtype=torch.bfloat16, device="cuda")
    ws.run(x.cuda(), scores.cuda(), torch.ones(E, dtype=torch.bfloat16, device="cuda"), table, y, rows, fp4=False)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert torch.all(y[rows * H:] == -3.0)
    capture = {}
    expected = omoe.forward(to_f32(x), to_f32(scores), np.ones(E, dtype=np.float32), host, mode="w4a16", capture=capture)
    assert np.array_equal(ws.selected_experts().cpu().numpy(), capture["ids"])
    assert_gemm_close(bits(ws.gate_up_capture()), C.bf16_bits(capture["gate_up"]), "W4A16 gate/up capture")
    assert_gemm_close(bits(ws.down_capture()), C.bf16_bits(capture["down"]), "W4A16 down capture")
    m = assert_gemm_close(bits(y[:rows * H].reshape(rows, H)), expected, f"W4A16 MoE rows={rows} {mode}")
    print(f"W4A16 rows={rows} {mode}: rel_fro {m['rel_fro']:.2e} max_abs/max {m['max_abs'] / m['max_ref']:.2e}")
    # the same table still runs with FP4 activations
    y4 = torch.empty((rows, H), dtype=torch.bfloat16, device="cuda")
    ws.run(x.cuda(), scores.cuda(), torch.ones(E, dtype=torch.bfloat16, device="cuda"), table, y4, rows, fp4=True)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0 and torch.isfinite(y4.float()).all()


@pytest.fixture(scope="module")
def experts_mixed(gw):
    """Every (expert, projection) with its own storage type, cycling BF16 / FP8 / NVFP4 as (expert + role) % 3
    (the fourth storage recipe of tests/gemma4_26b_moe_quantized.cu:104-118), all from the same N(0, 0.02)
    matrices; FP8 with per-tensor weight scale amax/448."""
    from oracle import fp8 as ofp8
    device, host = [], []
    for e in range(E):
        g = torch.Generator().manual_seed(9 * 1000 + e)
        shapes = [(I, H), (I, H), (H, I)]
        dev_row, host_row = [], []
        for role, (n, k) in enumerate(shapes):
            m = (torch.randn((n, k), generator=g) * 0.02).bfloat16()
            kind = (e + role) % 3
            input_scale = [0.004, 0.0045, 0.0007][role] * (1 + 0.1 * (e % 3))
            if kind == 0:
                dev_row.append(m.cuda())
                host_row.append(to_f32(m))
            elif kind == 1:
                hw = ofp8.pack_weights(to_f32(m), input_scale)
                dev_row.append(gw.Fp8Weight(torch.from_numpy(hw.data.copy()).cuda(), hw.input_scale, hw.weight_scale))
                host_row.append(hw)
            else:
                packed = pack_padded(gw, m.cuda(), input_scale, (n + 127) // 128 * 128)
                dev_row.append(packed)
                host_row.append(onv.Weight(packed.data.cpu().numpy(), packed.scales.cpu().numpy(), packed.input_scale,
                                           packed.weight_scale, packed.data.shape[0], k))
        device.append(tuple(dev_row))
        host.append(omoe.ExpertWeights(*host_row))
    return gw.ExpertTable(device), host


@pytest.mark.parametrize("rows,mode,fp4", [(1, "hot", True), (17, "distributed", True), (129, "uneven", True),
                                           (300, "normal", True), (700, "normal", True), (33, "normal", False),
                                           (600, "uneven", False)])
def test_moe_mixed_storage_vs_oracle(gw, experts_mixed, rows, mode, fp4):
    """BF16, FP8 and NVFP4 projections side by side in one table (tests/gemma4_26b_moe_quantized.cu:57-253
    runs six such recipes): each projection against the oracle of its own storage type -- FP32 matmul for
    BF16, the W8A8 oracle for FP8, W4A4 or (fp4 = 0) W4A16 for NVFP4."""
    table, host = experts_mixed
    if not fp4:
        table.enable_w4a16()
    x = bf16_normal((rows, H), 500 + rows)
    scores = make_scores(rows, mode, rows)
    ws = gw.MoeWorkspace(max(rows, 64), fp8_experts=True)
    y = torch.full((rows * H + 64,), -3.0, dtype=torch.bfloat16, device="cuda")
    ws.run(x.cuda(), scores.cuda(), torch.ones(E, dtype=torch.bfloat16, device="cuda"), table, y, rows,
           has_bf16=True, has_fp8=True, has_nvfp4=True, fp4=fp4)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert torch.all(y[rows * H:] == -3.0)
    capture = {}
    expected = omoe.forward(to_f32(x), to_f32(scores), np.ones(E, dtype=np.float32), host,
                            mode="w4a4" if fp4 else "w4a16", capture=capture, rcp_fn=gw.rcp_approx, gelu_fn=gw.geglu_bf16)
    assert np.array_equal(ws.selected_experts().cpu().numpy(), capture["ids"])
    assert_gemm_close(bits(ws.gate_up_capture()), C.bf16_bits(capture["gate_up"]), "mixed gate/up capture")
    assert_gemm_close(bits(ws.activated_capture()), C.bf16_bits(capture["activated"]), "mixed activated capture")
    assert_gemm_close(bits(ws.down_capture()), C.bf16_bits(capture["down"]), "mixed down capture")
    m = assert_gemm_close(bits(y[:rows * H].reshape(rows, H)), expected, f"mixed MoE rows={rows} {mode} fp4={fp4}")
    print(f"mixed rows={rows} {mode} fp4={fp4}: rel_fro {m['rel_fro']:.2e}")
    # a workspace without the FP8 staging refuses FP8 experts instead of computing garbage
    with pytest.raises(gw.GewellUnsupported, match="GW_MOE_FP8_EXPERTS"):
        gw.MoeWorkspace(4).run(x.cuda(), scores.cuda(), torch.ones(E, dtype=torch.bfloat16, device="cuda"), table, y, 1,
                               has_bf16=True, has_fp8=True, has_nvfp4=True, fp4=True)


_sampled_oracle_cache = {}


def _zipf_bias():
    ranks = torch.arange(1, E + 1, dtype=torch.float32)
    p = ranks.pow(-1.2)
    return (p / p.sum()).log()


@pytest.mark.parametrize("rows,form,skew", [(8192, None, False), (8192, "direct", False), (8192, "fused-single", False),
                                            (32768, None, True)])
def test_moe_layer_sampled_tokens_vs_oracle(gw, experts_shared, moe_form, rows, form, skew):
    """The published layer sizes (8192 tokens on one GPU; 32768 tokens with the Zipf(1.2) routing
    bias, the expert-parallel configuration's whole batch) against the faithful W4A4 oracle.  The
    layer is row independent (tests/gemma4_26b_moe_quantized.cu:57-253 checks it per row too), so
    the oracle evaluates a sample of tokens -- first, last and random ones -- with the routing it
    computes itself, and those rows of the full-size run must match."""
    table, host = experts_shared
    moe_form(form)
    x = bf16_normal((rows, H), 300 + rows % 97)
    scores = make_scores(rows, "normal", 12)
    if skew:
        scores = (scores.float() + _zipf_bias()).bfloat16()
    ws = gw.MoeWorkspace(rows)
    y = torch.empty((rows, H), dtype=torch.bfloat16, device="cuda")
    ws.run(x.cuda(), scores.cuda(), torch.ones(E, dtype=torch.bfloat16, device="cuda"), table, y, rows)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    rng = np.random.default_rng(rows)
    sample = np.unique(np.concatenate([[0, 1, 63, 64, rows - 1], rng.integers(0, rows, 19)]))
    key = (rows, skew)
    if key not in _sampled_oracle_cache:
        capture = {}
        expected = omoe.forward(to_f32(x[sample]), to_f32(scores[sample]), np.ones(E, dtype=np.float32), host,
                                capture=capture, rcp_fn=gw.rcp_approx, gelu_fn=gw.geglu_bf16)
        _sampled_oracle_cache[key] = (expected, capture["ids"])
    expected, ids = _sampled_oracle_cache[key]
    assert np.array_equal(ws.selected_experts().cpu().numpy()[sample], ids)
    m = assert_gemm_close(bits(y[torch.from_numpy(sample).cuda()]), expected, f"MoE rows={rows} form={form} sampled tokens")
    print(f"rows={rows} form={form}: {len(sample)} sampled tokens rel_fro {m['rel_fro']:.2e} "
          f"max_abs/max {m['max_abs'] / m['max_ref']:.2e}")


@pytest.mark.parametrize("rows", [100, 700])
def test_moe_quantised_input_bytes_exact(gw, experts, rows):
    """The gather + FP4 quantisation step (moe.cu:183-186,254-304) byte for byte: every sorted row is
    its token quantised with the destination expert's input scale, gate and up separately when their
    scales differ; scale bytes sit in the expert's 128-row aligned region in the tiled layout.  Both
    quantisers are covered: one thread per block (small batches) and one warp per token (from 512
    tokens on)."""
    table, host = experts
    x = bf16_normal((rows, H), 55)
    scores = make_scores(rows, "normal", 3)
    ws = gw.MoeWorkspace(rows)
    y = torch.empty((rows, H), dtype=torch.bfloat16, device="cuda")
    ws.run(x.cuda(), scores.cuda(), torch.ones(E, dtype=torch.bfloat16, device="cuda"), table, y, rows)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    packed, tiles = ws.quantized_input(parts=2)
    packed, tiles = packed.cpu().numpy(), tiles.cpu().numpy()
    order, offsets = ws.sorted_assignments().cpu().numpy(), ws.offsets().cpu().numpy()
    xf = to_f32(x)
    checked = 0
    for e in range(E):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if lo == hi:
            continue
        tokens = order[lo:hi] // 8
        region = (lo // 128 + e) * 128 * (H // 16)
        for part, weight in enumerate((host[e].gate, host[e].up)):
            q = onv.quantize_activations(xf[tokens], weight.input_scale, rcp_fn=gw.rcp_approx)
            assert np.array_equal(packed[part, lo:hi], q.packed[:hi - lo]), f"expert {e} part {part}: packed bytes"
            got = onv.untile_scales(tiles[part, region:region + onv.scale_storage_bytes(hi - lo, H)], hi - lo, H)
            assert np.array_equal(got, q.scales_linear), f"expert {e} part {part}: scale bytes"
            checked += hi - lo
    assert checked == 2 * 8 * rows
