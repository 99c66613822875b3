"""GPU parity of the dense MLP chain (gate + up projection -> GeGLU -> down projection of one 31B
layer, Executor::project_mlp, models/gemma4/31b/sm120/executor.cuh:1248-1291) through the C ABI, for
every route the weights' storage and layout can select: joined or separate gate/up, GeGLU fused into
the down projection's quantiser or as a kernel of its own, FP4 / FP8 / BF16 activations.  The oracle
composes the per-layer oracles of the linear layers."""
import numpy as np
import pytest
import torch

from oracle import codecs as C
from oracle import fp8 as ofp8
from oracle import nvfp4 as onv
from tests.gpu_helpers import assert_gemm_close, bf16_normal, bits, device_weight_to_oracle, to_f32

pytestmark = pytest.mark.gpu

H, M = 512, 384


@pytest.fixture(scope="module")
def gw():
    import gewell_b200
    return gewell_b200


def nvfp4_layer(gw, joined: bool, x_amax: float):
    """gate / up / down as NVFP4; joined: gate and up packed as one [2M, H] matrix (one global scale, rows
    and scale tiles back to back, one input scale), else packed apart with different input scales."""
    wgu = bf16_normal((2 * M, H), 1, 0.05).cuda()
    wd = bf16_normal((H, M), 2, 0.05).cuda()
    down = gw.nvfp4_pack_weights(wd, 0.004)
    if joined:
        both = gw.nvfp4_pack_weights(wgu, x_amax / 2688)
        split = gw.nvfp4_scale_storage_bytes(M, H)
        gate = gw.Nvfp4Weight(both.data[:M], both.scales[:split], both.input_scale, both.weight_scale)
        up = gw.Nvfp4Weight(both.data[M:], both.scales[split:], both.input_scale, both.weight_scale)
        keep = both
    else:
        gate = gw.nvfp4_pack_weights(wgu[:M].contiguous(), x_amax / 2688)
        up = gw.nvfp4_pack_weights(wgu[M:].contiguous(), x_amax / 2000)
        keep = None
    return gate, up, down, keep


def oracle_nvfp4_chain(x, gate, up, down, fp4, gw):
    hg, hu, hd = (device_weight_to_oracle(w, n, k) for w, n, k in ((gate, M, H), (up, M, H), (down, H, M)))
    if fp4:
        g = C.bf16_to_f32(onv.linear_w4a4(x, hg, rcp_fn=gw.rcp_approx))
        u = C.bf16_to_f32(onv.linear_w4a4(x, hu, rcp_fn=gw.rcp_approx))
        act = gw.geglu_bf16(g, u)
        return onv.linear_w4a4(act, hd, rcp_fn=gw.rcp_approx)
    g = C.bf16_to_f32(onv.linear_w4a16(x, hg))
    u = C.bf16_to_f32(onv.linear_w4a16(x, hu))
    return onv.linear_w4a16(C.gelu_tanh_multiply_bf16(g, u), hd)


@pytest.mark.parametrize("rows", [5, 200])
@pytest.mark.parametrize("joined", [True, False])
@pytest.mark.parametrize("policy,phase", [("always", "decode"), ("prefill", "prefill"), ("prefill", "decode")])
def test_nvfp4_mlp_chain(gw, rows, joined, policy, phase):
    from gewell_b200 import _lib
    x = bf16_normal((rows, H), 3)
    gate, up, down, _keep = nvfp4_layer(gw, joined, float(np.abs(to_f32(x)).max()))
    chain = gw.MlpChain(H, M, 256, getattr(_lib, "POLICY_" + policy.upper()))
    nbytes = chain.bytes()
    chain.prepare(rows)
    projections = [gw.make_projection(w, k, n) for w, k, n in ((gate, H, M), (up, H, M), (down, M, H))]
    for p in projections:
        p.physical_output = p.output            # 31B matrices are not padded (their widths divide by 128)
    y = chain.run(*projections, x.cuda(), getattr(_lib, "PHASE_" + phase.upper()))
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0 and chain.bytes() == nbytes
    fp4 = policy == "always" or phase == "prefill"
    expected = oracle_nvfp4_chain(to_f32(x), gate, up, down, fp4, gw)
    m = assert_gemm_close(bits(y), expected, f"NVFP4 MLP chain rows={rows} joined={joined} {policy}/{phase}")
    print(f"rows={rows} joined={joined} {policy}/{phase}: rel_fro {m['rel_fro']:.2e}")


@pytest.mark.parametrize("rows", [3, 160])
@pytest.mark.parametrize("joined", [True, False])
def test_fp8_mlp_chain(gw, rows, joined):
    from gewell_b200 import _lib
    x = bf16_normal((rows, H), 4)
    xs = float(np.abs(to_f32(x)).max() / 448)
    wgu, wd = to_f32(bf16_normal((2 * M, H), 5, 0.05)), to_f32(bf16_normal((H, M), 6, 0.05))
    hd = ofp8.pack_weights(wd, 0.02)
    down = gw.Fp8Weight(torch.from_numpy(hd.data.copy()).cuda(), hd.input_scale, hd.weight_scale)
    if joined:
        hgu = ofp8.pack_weights_per_channel(wgu, xs)
        data = torch.from_numpy(hgu.data.copy()).cuda()
        channel = torch.from_numpy(hgu.channel_scales.copy()).cuda()
        gate = gw.Fp8Weight(data[:M], xs, 1.0, channel[:M])
        up = gw.Fp8Weight(data[M:], xs, 1.0, channel[M:])
        gu = C.bf16_to_f32(ofp8.linear_w8a8(to_f32(x), hgu))
        g, u = gu[:, :M], gu[:, M:]
    else:
        hg, hu = ofp8.pack_weights(wgu[:M], xs), ofp8.pack_weights(wgu[M:], xs * 1.5)
        gate = gw.Fp8Weight(torch.from_numpy(hg.data.copy()).cuda(), hg.input_scale, hg.weight_scale)
        up = gw.Fp8Weight(torch.from_numpy(hu.data.copy()).cuda(), hu.input_scale, hu.weight_scale)
        g = C.bf16_to_f32(ofp8.linear_w8a8(to_f32(x), hg))
        u = C.bf16_to_f32(ofp8.linear_w8a8(to_f32(x), hu))
    expected = ofp8.linear_w8a8(gw.geglu_bf16(g, u), hd)
    chain = gw.MlpChain(H, M, 256, _lib.POLICY_ALWAYS)
    chain.prepare(rows)
    y = chain.run(gw.make_projection(gate, H, M), gw.make_projection(up, H, M), gw.make_projection(down, M, H), x.cuda(),
                  _lib.PHASE_DECODE)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert_gemm_close(bits(y), expected, f"FP8 MLP chain rows={rows} joined={joined}")


@pytest.mark.parametrize("rows", [2, 130])
@pytest.mark.parametrize("joined", [True, False])
def test_bf16_mlp_chain(gw, rows, joined):
    from gewell_b200 import _lib
    x = bf16_normal((rows, H), 7)
    wgu, wd = bf16_normal((2 * M, H), 8, 0.05).cuda(), bf16_normal((H, M), 9, 0.05).cuda()
    gate, up = (wgu[:M], wgu[M:]) if joined else (wgu[:M].clone(), wgu[M:].clone())
    chain = gw.MlpChain(H, M, 256, _lib.POLICY_ALWAYS)
    chain.prepare(rows)
    y = chain.run(gw.make_projection(gate, H, M), gw.make_projection(up, H, M), gw.make_projection(wd, M, H), x.cuda(),
                  _lib.PHASE_PREFILL)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    g = C.bf16_round(to_f32(x) @ to_f32(wgu[:M]).T)
    u = C.bf16_round(to_f32(x) @ to_f32(wgu[M:]).T)
    expected = C.bf16_bits(C.gelu_tanh_multiply_bf16(g, u) @ to_f32(wd).T)
    assert_gemm_close(bits(y), expected, f"BF16 MLP chain rows={rows} joined={joined}")


def test_mlp_chain_validation(gw):
    from gewell_b200 import _lib
    with pytest.raises(gw.GewellInvalidArgument):
        gw.MlpChain(500, M, 8, _lib.POLICY_ALWAYS)
    chain = gw.MlpChain(H, M, 8, _lib.POLICY_ALWAYS)
    w = bf16_normal((M, H), 1).cuda()
    p = gw.make_projection(w, H, M)
    with pytest.raises(gw.GewellInvalidArgument):      # run before prepare
        chain.rows = 4
        chain.run(p, p, gw.make_projection(bf16_normal((H, M), 2).cuda(), M, H), bf16_normal((4, H), 3).cuda(), 0)


# ------------------------------------------------------------------------------------------------
# Attention input projections (Executor::project_qkv, executor.cuh:1218-1247) and the loader's joins
# (weights.cuh:146-223)

Q, KV = 256, 128


@pytest.mark.parametrize("rows", [3, 150])
@pytest.mark.parametrize("with_value", [True, False])
@pytest.mark.parametrize("adjacent", [True, False])
def test_qkv_bf16(gw, rows, with_value, adjacent):
    from gewell_b200 import _lib
    x = bf16_normal((rows, H), 11)
    w = bf16_normal((Q + 2 * KV, H), 12, 0.05).cuda()
    parts = [w[:Q], w[Q:Q + KV], w[Q + KV:]]
    if not adjacent:                                 # the same matrices with 128 bytes between them
        spaced = torch.zeros((Q + 2 * KV) * H + 3 * 64, dtype=torch.bfloat16, device="cuda")
        starts = [0, Q * H + 64, (Q + KV) * H + 128]
        parts = [spaced[s0:s0 + p.numel()].view(p.shape).copy_(p) for s0, p in zip(starts, parts)]
    projector = gw.QkvProjector(H, Q, KV, 256, _lib.POLICY_ALWAYS)
    projector.prepare(rows)
    bound = [gw.make_projection(p, H, p.shape[0]) for p in parts]
    q, k, v, joined = projector.run(bound[0], bound[1], bound[2] if with_value else None, x.cuda(), _lib.PHASE_DECODE)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0 and joined == adjacent
    for name, got, weight in (("q", q, parts[0]), ("k", k, parts[1]), ("v", v, parts[2])):
        if got is None:
            assert name == "v" and not with_value
            continue
        expected = C.bf16_bits(to_f32(x) @ to_f32(weight).T)
        assert_gemm_close(bits(got.contiguous()), expected, f"BF16 {name} rows={rows} adjacent={adjacent}")


def test_fp8_group_join_then_joined_qkv(gw):
    """Three FP8 matrices with their own weight scales and 8-byte trailers between them, as an artifact holds
    them: separate projections before the join, one channel-scaled GEMM after it, same results."""
    from gewell_b200 import _lib
    rows = 40
    x = bf16_normal((rows, H), 13)
    xs = float(np.abs(to_f32(x)).max() / 448)
    shapes = [Q, KV, KV]
    host = [ofp8.pack_weights(to_f32(bf16_normal((n, H), 20 + i, 0.05)), xs) for i, n in enumerate(shapes)]
    region = torch.zeros(sum(n * H + 256 for n in shapes), dtype=torch.uint8, device="cuda")
    group = (_lib.Projection * 3)()
    offset = 0
    for p, h, n in zip(group, host, shapes):
        region[offset:offset + n * H] = torch.from_numpy(h.data.copy()).cuda().reshape(-1)
        p.storage, p.input, p.output, p.physical_output = _lib.STORAGE_FP8_W8A8, H, n, n
        p.fp8_data = region.data_ptr() + offset
        p.fp8_input_scale, p.fp8_weight_scale = h.input_scale, h.weight_scale
        offset += n * H + 256                       # trailer and alignment padding
    projector = gw.QkvProjector(H, Q, KV, 64, _lib.POLICY_ALWAYS)
    projector.prepare(rows)
    before = projector.run(group[0], group[1], group[2], x.cuda(), _lib.PHASE_PREFILL)
    assert before[3] is False
    before = [t.clone() for t in before[:3]]
    channel = torch.zeros(sum(shapes), dtype=torch.float32, device="cuda")
    assert gw.join_fp8_group(group, channel)
    assert group[1].fp8_data == group[0].fp8_data + Q * H and group[2].fp8_data == group[1].fp8_data + KV * H
    expected_scales = np.concatenate([np.full(n, np.float32(h.input_scale) * np.float32(h.weight_scale), dtype=np.float32)
                                      for h, n in zip(host, shapes)])
    assert np.array_equal(channel.cpu().numpy(), expected_scales)
    q, k, v, joined = projector.run(group[0], group[1], group[2], x.cuda(), _lib.PHASE_PREFILL)
    torch.cuda.synchronize()
    assert joined and gw.kernel_error() == 0
    for got, old, h in zip((q, k, v), before, host):
        expected = ofp8.linear_w8a8(to_f32(x), h)
        assert_gemm_close(bits(got.contiguous()), expected, "FP8 joined QKV")
        assert_gemm_close(bits(got.contiguous()), bits(old), "FP8 joined vs separate")
    # different input scales: the group is left apart
    group[1].fp8_input_scale = xs * 2
    assert not gw.join_fp8_group(group, channel)


def test_nvfp4_pair_join_in_place(gw):
    """Gate and up payloads apart in one region (rows, scale tiles, trailer each) -> joined in place; the chain
    then runs the joined GEMM and gives the bits of a layer packed jointly from the start."""
    from gewell_b200 import _lib
    rows = 70
    x = bf16_normal((rows, H), 14)
    gate, up, down, both = nvfp4_layer(gw, True, float(np.abs(to_f32(x)).max()))
    packed, scales = M * H // 2, gw.nvfp4_scale_storage_bytes(M, H)
    stride = packed + scales + 256
    region = torch.zeros(2 * stride, dtype=torch.uint8, device="cuda")
    bound = []
    for i, w in enumerate((gate, up)):
        region[i * stride:i * stride + packed] = w.data.reshape(-1)
        region[i * stride + packed:i * stride + packed + scales] = w.scales.reshape(-1)
        p = gw.make_projection(w, H, M)
        p.physical_output = M
        p.nvfp4_data = region.data_ptr() + i * stride
        p.nvfp4_scales = region.data_ptr() + i * stride + packed
        bound.append(p)
    p_down = gw.make_projection(down, M, H)
    p_down.physical_output = H
    chain = gw.MlpChain(H, M, 128, _lib.POLICY_ALWAYS)
    chain.prepare(rows)
    apart = chain.run(bound[0], bound[1], p_down, x.cuda(), _lib.PHASE_PREFILL).clone()
    assert gw.join_nvfp4_pair(bound[0], bound[1])
    assert bound[1].nvfp4_data == bound[0].nvfp4_data + packed
    assert bound[0].nvfp4_scales == bound[0].nvfp4_data + 2 * packed and bound[1].nvfp4_scales == bound[0].nvfp4_scales + scales
    assert torch.equal(region[:2 * packed].view(2 * M, H // 2), both.data)
    assert torch.equal(region[2 * packed:2 * (packed + scales)], both.scales.reshape(-1))
    together = chain.run(bound[0], bound[1], p_down, x.cuda(), _lib.PHASE_PREFILL)
    reference_bound = [gw.make_projection(w, H, M) for w in (gate, up)]
    for p in reference_bound:
        p.physical_output = M
    expected = chain.run(reference_bound[0], reference_bound[1], p_down, x.cuda(), _lib.PHASE_PREFILL)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert torch.equal(together, expected)
    assert_gemm_close(bits(together), bits(apart), "joined vs apart")
    # different weight scales: left apart
    bound[1].nvfp4_weight_scale *= 2
    assert not gw.join_nvfp4_pair(bound[0], bound[1])
