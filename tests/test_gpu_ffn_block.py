"""GPU parity of the feed-forward block of a 26B-A4B layer around the MoE (three-output RMS norm,
shared MLP, router projection, MoE, post norms, residual adds, layer scalar:
models/gemma4/26b_a4b/sm120/batched_executor.cu:250-286, bf16_math.cuh:17-117) through the C ABI.

The norms, adds and the scalar are compared bit for bit with the CPU oracle (oracle/ffn.py), which gets the
device's rsqrtf values where it needs that approximate instruction; a second comparison with the host's
correctly rounded 1/sqrt bounds what that instruction can change (rare one-ulp flips)."""
import numpy as np
import pytest
import torch

from oracle import codecs as C
from oracle import ffn as offn
from oracle import fp8 as ofp8
from oracle import moe as omoe
from oracle import nvfp4 as onv
from tests.gpu_helpers import assert_gemm_close, bf16_normal, bits, device_weight_to_oracle, to_f32
from tests.test_gpu_moe import experts, experts_shared, make_scores, pack_padded  # noqa: F401  (fixtures)

pytestmark = pytest.mark.gpu

H, S, E = 2816, 2112, 128


@pytest.fixture(scope="module")
def gw():
    import gewell_b200
    return gewell_b200


def norm_weight(seed, width=H):
    return (1.0 + 0.25 * bf16_normal((width,), seed).float()).to(torch.bfloat16)


def ulp_distance(actual_bits, expected_bits):
    def key(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, 0x8000 - b, b)
    return np.abs(key(actual_bits) - key(expected_bits))


@pytest.mark.parametrize("rows,width", [(1, H), (2, H), (3, H), (4, H), (8, H), (16, H), (33, H), (300, H),
                                        (5, 64), (40, 256), (7, 512), (2, 8), (1, 16384)])
@pytest.mark.parametrize("weighted", [True, False])
def test_rms_norm_bit_exact(gw, rows, width, weighted):
    """Every reduction order the launch rule selects (512 ... 32 lanes at the layer's width, fewer at small
    widths), with and without a weight."""
    from gewell_b200 import _lib
    assert _lib.load().gw_rms_norm_reduction_lanes(rows, width) == offn.reduction_lanes(rows, width)
    x = bf16_normal((rows, width), 10 + rows, 3.0)
    x[0, :4] = torch.tensor([0.0, -0.0, 2.0 ** -120, 3.0e4], dtype=torch.bfloat16)
    w = norm_weight(3, width) if weighted else None
    y = gw.rms_norm(x.cuda(), None if w is None else w.cuda())
    torch.cuda.synchronize()
    wf = None if w is None else to_f32(w)
    exact = offn.rms_norm(to_f32(x), wf, rsqrt_fn=gw.rsqrt_device)
    assert np.array_equal(bits(y), C.bf16_bits(exact))
    host = C.bf16_bits(offn.rms_norm(to_f32(x), wf))
    distance = ulp_distance(bits(y), host)
    assert distance.max() <= 1 and np.mean(distance != 0) < 0.01


def test_zero_row_and_validation(gw):
    x = torch.zeros((2, 64), dtype=torch.bfloat16, device="cuda")
    y = gw.rms_norm(x)
    assert torch.all(y == 0)                       # rsqrt(1e-6) * 0
    with pytest.raises(gw.GewellInvalidArgument):
        gw.rms_norm(torch.zeros((2, 12), dtype=torch.bfloat16, device="cuda"))
    gw.rms_norm(torch.zeros((0, 64), dtype=torch.bfloat16, device="cuda"))      # rows == 0: no-op


@pytest.mark.parametrize("rows", [1, 6, 16, 129])
def test_feedforward_norm_bit_exact(gw, rows):
    x = bf16_normal((rows, H), 20 + rows, 2.0)
    ws, wr, we = norm_weight(4), norm_weight(5), norm_weight(6)
    shared, router, expert = gw.rms_norm_feedforward(x.cuda(), ws.cuda(), wr.cuda(), we.cuda())
    torch.cuda.synchronize()
    es, er, ee = offn.rms_norm_feedforward(to_f32(x), to_f32(ws), to_f32(wr), to_f32(we), rsqrt_fn=gw.rsqrt_device)
    assert np.array_equal(bits(shared), C.bf16_bits(es))
    assert np.array_equal(bits(router), C.bf16_bits(er))
    assert np.array_equal(bits(expert), C.bf16_bits(ee))
    # the shared and expert outputs are plain norms with their own weights
    assert torch.equal(shared, gw.rms_norm(x.cuda(), ws.cuda()))
    assert torch.equal(expert, gw.rms_norm(x.cuda(), we.cuda()))


def test_add_and_scale_bit_exact(gw):
    a, b = bf16_normal((37, 100), 1, 50.0), bf16_normal((37, 100), 2, 0.01)
    a[0, :3] = torch.tensor([3.0e38, -3.0e38, 1.0], dtype=torch.bfloat16)
    b[0, :3] = torch.tensor([3.0e38, 3.0e38, 2.0 ** -9], dtype=torch.bfloat16)
    y = gw.add_bf16(a.cuda(), b.cuda())
    assert np.array_equal(bits(y), C.bf16_bits(offn.add(to_f32(a), to_f32(b))))
    scalar = torch.tensor([0.7109375], dtype=torch.bfloat16)
    z = gw.scale_bf16(a.clone().cuda(), scalar.cuda())
    assert np.array_equal(bits(z), C.bf16_bits(offn.scale(to_f32(a), float(scalar))))


@pytest.mark.parametrize("rows", [1, 5, 16, 200])
def test_tail_equals_the_seven_steps(gw, rows):
    """The one-launch tail against its parts run one by one (bit for bit) and against the oracle."""
    hidden = bf16_normal((rows, H), 31, 4.0)
    shared_mlp, routed = bf16_normal((rows, H), 32, 0.7), bf16_normal((rows, H), 33, 1.5)
    w1, w2, w3 = norm_weight(7), norm_weight(8), norm_weight(9)
    scalar = torch.tensor([0.8203125], dtype=torch.bfloat16)
    fused = gw.ffn_tail(shared_mlp.cuda(), routed.cuda(), w1.cuda(), w2.cuda(), w3.cuda(), scalar.cuda(), hidden.clone().cuda())
    shared = gw.rms_norm(shared_mlp.cuda(), w1.cuda())
    branch = gw.rms_norm(routed.cuda(), w2.cuda())
    shared = gw.add_bf16(shared, branch)
    branch = gw.rms_norm(shared, w3.cuda())
    stepwise = gw.scale_bf16(gw.add_bf16(hidden.cuda(), branch), scalar.cuda())
    torch.cuda.synchronize()
    assert torch.equal(fused, stepwise)
    expected = offn.tail(to_f32(hidden), to_f32(shared_mlp), to_f32(routed), to_f32(w1), to_f32(w2), to_f32(w3),
                         float(scalar), rsqrt_fn=gw.rsqrt_device)
    assert np.array_equal(bits(fused), C.bf16_bits(expected))


def shared_mlp_weights(gw, storage):
    wg, wu, wd = bf16_normal((S, H), 41, 0.02), bf16_normal((S, H), 42, 0.02), bf16_normal((H, S), 43, 0.02)
    if storage == "bf16":
        device = [wg.cuda(), wu.cuda(), wd.cuda()]
        return device, [to_f32(wg), to_f32(wu), to_f32(wd)]
    if storage == "fp8":
        host = [ofp8.pack_weights(to_f32(w), s) for w, s in ((wg, 0.01), (wu, 0.012), (wd, 0.004))]
        return [gw.Fp8Weight(torch.from_numpy(h.data.copy()).cuda(), h.input_scale, h.weight_scale) for h in host], host
    device = [pack_padded(gw, w.cuda(), s, (w.shape[0] + 127) // 128 * 128) for w, s in ((wg, 0.0017), (wu, 0.0019), (wd, 0.0006))]
    host = [onv.Weight(p.data.cpu().numpy(), p.scales.cpu().numpy(), p.input_scale, p.weight_scale, p.data.shape[0], w.shape[1])
            for p, w in zip(device, (wg, wu, wd))]
    return device, host


def oracle_shared_mlp(gw, normalized, host, storage, fp4):
    def project(x, w, logical):
        if storage == "bf16":
            return C.bf16_round(x @ w.T)
        if storage == "fp8":
            return C.bf16_to_f32(ofp8.linear_w8a8(x, w))
        if fp4:
            return C.bf16_to_f32(onv.linear_w4a4(x, w, rcp_fn=gw.rcp_approx))[:, :logical]
        return C.bf16_to_f32(onv.linear_w4a16(x, w, logical))
    gate, up = project(normalized, host[0], S), project(normalized, host[1], S)
    return project(gw.geglu_bf16(gate, up), host[2], H)


@pytest.mark.parametrize("rows,storage,policy,phase", [
    (5, "nvfp4", "always", "decode"), (200, "nvfp4", "always", "prefill"), (300, "fp8", "always", "prefill"),
    (16, "bf16", "always", "decode"), (40, "nvfp4", "prefill", "decode")])
def test_ffn_block_stage_by_stage(gw, experts_shared, rows, storage, policy, phase):
    """One layer's block.  Every stage is checked against the oracle fed with the device's previous stage
    (as the reference's capture-based checks do): norms and tail bit for bit, GEMM stages at the
    path's GEMM tolerance, routing ids exactly."""
    from gewell_b200 import _lib
    table, host_experts = experts_shared
    fp4 = policy == "always" or phase == "prefill"
    if not fp4:
        table.enable_w4a16()
    device_mlp, host_mlp = shared_mlp_weights(gw, storage)
    names = ("pre_feedforward_norm", "router_scale", "pre_feedforward_norm_2", "post_feedforward_norm_1",
             "post_feedforward_norm_2", "post_feedforward_norm")
    norms = {name: norm_weight(50 + i) for i, name in enumerate(names)}
    layer_scalar = torch.tensor([0.8984375], dtype=torch.bfloat16)
    router_proj = bf16_normal((E, H), 60, 0.5)
    per_expert = (1.0 + 0.1 * torch.sin(torch.arange(E, dtype=torch.float32))).to(torch.bfloat16)
    layer = {name: w.cuda() for name, w in norms.items()}
    layer.update(layer_scalar=layer_scalar.cuda(), router_proj=router_proj.cuda(), router_per_expert_scale=per_expert.cuda(),
                 gate=device_mlp[0], up=device_mlp[1], down=device_mlp[2], experts=table)
    block = gw.FfnBlock([layer], max(rows, 64), getattr(_lib, "POLICY_" + policy.upper()))
    nbytes = block.bytes()
    block.prepare(rows, getattr(_lib, "PHASE_" + phase.upper()))
    hidden0 = bf16_normal((rows, H), 70 + rows, 2.0)
    hidden = block.run(0, hidden0.clone().cuda())
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0 and block.bytes() == nbytes
    f = {name: to_f32(w) for name, w in norms.items()}
    # 1. the three-output norm, bit for bit
    es, er, ee = offn.rms_norm_feedforward(to_f32(hidden0), f["pre_feedforward_norm"], f["router_scale"],
                                           f["pre_feedforward_norm_2"], rsqrt_fn=gw.rsqrt_device)
    normalized, router_input, expert_input = block.buffer("normalized"), block.buffer("router_input"), block.buffer("expert_input")
    assert np.array_equal(bits(normalized), C.bf16_bits(es))
    assert np.array_equal(bits(router_input), C.bf16_bits(er))
    assert np.array_equal(bits(expert_input), C.bf16_bits(ee))
    # 2. shared MLP and router logits from the device's norm outputs
    shared_mlp = block.buffer("shared_mlp")
    expected_mlp = oracle_shared_mlp(gw, to_f32(normalized), host_mlp, storage, fp4)
    m_mlp = assert_gemm_close(bits(shared_mlp), C.bf16_bits(expected_mlp), f"shared MLP {storage}")
    logits = block.buffer("router_logits")
    m_router = assert_gemm_close(bits(logits), C.bf16_bits(to_f32(router_input) @ to_f32(router_proj).T), "router logits")
    # 3. the MoE layer from the device's logits and expert input
    routed = block.buffer("routed")
    capture = {}
    expected_routed = omoe.forward(to_f32(expert_input), to_f32(logits), to_f32(per_expert), host_experts,
                                   mode="w4a4" if fp4 else "w4a16", capture=capture, rcp_fn=gw.rcp_approx,
                                   gelu_fn=gw.geglu_bf16 if fp4 else None)
    assert np.array_equal(block.selected_experts().cpu().numpy(), capture["ids"])
    m_moe = assert_gemm_close(bits(routed), expected_routed, "routed experts")
    # 4. the tail from the device's two branches, bit for bit
    expected = offn.tail(to_f32(hidden0), to_f32(shared_mlp), to_f32(routed), f["post_feedforward_norm_1"],
                         f["post_feedforward_norm_2"], f["post_feedforward_norm"], float(layer_scalar),
                         rsqrt_fn=gw.rsqrt_device)
    assert np.array_equal(bits(hidden), C.bf16_bits(expected))
    print(f"rows={rows} {storage} {policy}/{phase}: shared MLP {m_mlp['rel_fro']:.2e} router {m_router['rel_fro']:.2e} "
          f"MoE {m_moe['rel_fro']:.2e}")


def test_ffn_block_validation(gw, experts_shared):
    from gewell_b200 import _lib
    table, _ = experts_shared
    w = norm_weight(1).cuda()
    layer = dict(pre_feedforward_norm=w, router_scale=w, pre_feedforward_norm_2=w, post_feedforward_norm_1=w,
                 post_feedforward_norm_2=w, post_feedforward_norm=w, layer_scalar=w[:1], router_proj=bf16_normal((E, H), 2).cuda(),
                 router_per_expert_scale=w[:E], gate=bf16_normal((S, H), 3).cuda(), up=bf16_normal((S, H), 4).cuda(),
                 down=bf16_normal((H, S), 5).cuda(), experts=table)
    block = gw.FfnBlock([layer], 8, _lib.POLICY_ALWAYS)
    with pytest.raises(gw.GewellInvalidArgument):          # run before prepare
        block.run(0, torch.zeros((4, H), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(gw.GewellInvalidArgument):          # more rows than the block holds
        block.prepare(9, _lib.PHASE_DECODE)
