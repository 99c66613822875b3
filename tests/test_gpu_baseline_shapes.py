"""GPU parity at the full shapes of the published configurations, where a whole
CPU oracle pass would take minutes: the projection runs at full size through
the C ABI and a sample of its outputs (tile corners, first and last tiles,
first and last waves of the persistent schedule, random positions) is compared
with the FP64 dot over the operands exactly as the device quantised them --
the reference's own linear oracle (tests/nvfp4_linear_test.cu:263-293) -- and,
for FP8, tests/fp8_linear_test.cu:95-117.  Full-shape rows of the reference's
regression grid: tests/nvfp4_linear_test.cu:394-420, tests/fp8_linear_test.cu:355-380.
"""
import numpy as np
import pytest
import torch

from oracle import codecs as C
from oracle import nvfp4 as onv
from tests.gpu_helpers import assert_reference_tolerance, bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gw():
    import gewell_b200
    return gewell_b200


def device_normal(shape, seed, std):
    """BF16 ~ N(0, std) generated on the device in row chunks (the full-size operands would take
    gigabytes as FP32 on the host; the oracle reads back what the device holds anyway)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
    step = max(1, (64 << 20) // shape[1])
    for r in range(0, shape[0], step):
        rows = min(step, shape[0] - r)
        out[r:r + rows] = (torch.randn((rows, shape[1]), generator=g, device="cuda") * std).bfloat16()
    return out


def sample_positions(extent, tile, count, rng):
    """Indices that cover every kind of place inside a tiling of `extent` by `tile`: the first and
    last element of the first, second and last tiles, plus random ones."""
    chosen = {0, 1, tile - 1, tile, 2 * tile - 1, extent - tile, extent - 1, extent - tile - 1, extent // 2}
    chosen = {i for i in chosen if 0 <= i < extent}
    while len(chosen) < min(count, extent):
        chosen.add(int(rng.integers(0, extent)))
    return np.array(sorted(chosen), dtype=np.int64)


def gather_tiled_scales(tiled: torch.Tensor, rows: np.ndarray, width: int) -> np.ndarray:
    """Linear [len(rows), width/16] scale bytes of the given rows out of tiled device storage."""
    blocks = np.arange(width // 16)
    offsets = onv.scale_offset(rows[:, None], blocks[None, :], width)
    return tiled[torch.from_numpy(offsets.reshape(-1)).cuda()].cpu().numpy().reshape(len(rows), width // 16)


def decoded_rows(packed_rows: np.ndarray, scale_rows: np.ndarray) -> np.ndarray:
    """E2M1 value x E4M3 block scale of whole rows, as FP64."""
    values = C.e2m1_decode(C.unpack_nibbles(packed_rows)).astype(np.float64)
    scales = C.e4m3_decode(scale_rows).astype(np.float64)
    return (values.reshape(values.shape[0], -1, 16) * scales[:, :, None]).reshape(values.shape)


def check_nvfp4_sample(gw, rows, k, n, seed, what, row_tile=128, channel_tile=256):
    weight = gw.nvfp4_pack_weights(device_normal((n, k), seed, 0.02))
    x = device_normal((rows, k), seed + 100, 1.0)
    weight.input_scale = float(x.float().abs().max() / 2688)
    plan = gw.Nvfp4Plan(rows, k, n)
    need = plan.scratch_bytes()
    assert need <= gw.lib.gw_nvfp4_scratch_upper_bound_bytes(rows, k, n)
    scratch = torch.full((need + 256,), 0xCD, dtype=torch.uint8, device="cuda")
    y = torch.full((rows * n + 128,), -7.0, dtype=torch.bfloat16, device="cuda")
    plan.run(x, weight, y, scratch, need)
    torch.cuda.synchronize()
    assert gw.kernel_error() == 0
    assert torch.all(scratch[need:] == 0xCD), "wrote beyond the scratch"
    assert torch.all(y[rows * n:] == -7.0), "wrote beyond the output"
    out = y[:rows * n].reshape(rows, n)
    assert torch.isfinite(out.float()).all()
    rng = np.random.default_rng(seed)
    r = sample_positions(rows, row_tile, 64, rng)
    c = sample_positions(n, channel_tile, 512, rng)
    packed = scratch[:rows * k // 2].reshape(rows, k // 2)[torch.from_numpy(r).cuda()].cpu().numpy()
    scale_base = (rows * k // 2 + 255) // 256 * 256
    act_scales = gather_tiled_scales(scratch[scale_base:scale_base + onv.scale_storage_bytes(rows, k)], r, k)
    a = decoded_rows(packed, act_scales)
    w = decoded_rows(weight.data[torch.from_numpy(c).cuda()].cpu().numpy(), gather_tiled_scales(weight.scales, c, k))
    alpha = np.float32(np.float32(weight.input_scale) * np.float32(weight.weight_scale))
    expected = C.bf16_bits(((a @ w.T) * np.float64(alpha)).astype(np.float32))
    got = bits(out[torch.from_numpy(r).cuda()][:, torch.from_numpy(c).cuda()])
    assert_reference_tolerance(got, expected, what)
    return out


@pytest.mark.parametrize("pair", [True, False])
def test_config3_full_shape(gw, pair, monkeypatch):
    """NVFP4 prefill down projection, 4096 x 21504 -> 5376: 84 ring stages per tile (the phase bits of
    every barrier wrap dozens of times) and 4.54 waves of tiles, on the CTA-pair kernel and on the
    single-CTA kernel."""
    if not pair:
        monkeypatch.setenv("GW_DENSE_NO_PAIR", "1")
    check_nvfp4_sample(gw, 4096, 21504, 5376, 3, f"config 3 full shape, pair={pair}")


@pytest.mark.parametrize("rows", [1024, 2048])
def test_nvfp4_gate_up_full_width(gw, rows):
    """The joined gate+up projection of the 31B model, 5376 -> 43008."""
    check_nvfp4_sample(gw, rows, 5376, 43008, 5, f"NVFP4 5376->43008 rows={rows}")


@pytest.mark.parametrize("rows", [129, 513, 2592])
def test_nvfp4_down_projection_row_grid(gw, rows):
    """Rows of the reference's regression grid around tile boundaries at the full (21504 -> 5376) shape."""
    check_nvfp4_sample(gw, rows, 21504, 5376, 6, f"NVFP4 21504->5376 rows={rows}")
