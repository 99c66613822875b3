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
