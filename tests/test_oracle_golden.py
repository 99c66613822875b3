"""The CPU oracle against the reference's golden vectors and against outputs
of the reference's own Python packers (tests/golden/reference_packers.npz,
made by tests/golden/make_golden.py)."""
import json

import numpy as np
import pytest

from oracle import codecs as C
from oracle import fp8, nvfp4


@pytest.fixture(scope="module")
def vectors(golden_dir):
    return json.loads((golden_dir / "reference_vectors.json").read_text())


@pytest.fixture(scope="module")
def packers(golden_dir):
    return np.load(golden_dir / "reference_packers.npz")


def words(hex_list):
    return np.array([int(w, 16) for w in hex_list], dtype=np.uint16)


def test_scalar_known_answers(vectors):
    k = vectors["scalar_kats"]
    for value, expected in k["round_e4m3"]:
        assert C.e4m3_round(np.float32(value)) == np.float32(expected)
    for value, expected in k["round_e2m1"]:
        assert C.e2m1_round(np.float32(value)) == np.float32(expected)
    for amax, g, expected in k["nvfp4_block_scale"]:
        assert nvfp4.block_scale(np.float32(amax), g) == np.float32(expected)


def test_fp8_qdq_golden(vectors):
    g = vectors["fp8_qdq"]
    assert np.array_equal(fp8.qdq(words(g["input_words"])), words(g["output_words"]))


def test_nvfp4_qdq_golden(vectors):
    g = vectors["nvfp4_qdq"]
    inp = np.zeros(g["length"], dtype=np.uint16)
    out = np.zeros(g["length"], dtype=np.uint16)
    for i, w in g["input_words"].items():
        inp[int(i)] = int(w, 16)
    for i, w in g["output_words"].items():
        out[int(i)] = int(w, 16)
    assert np.array_equal(nvfp4.qdq(inp), out)


def test_vllm_activation_fixtures(vectors):
    """The two frozen scaled_fp4_quant outputs must be reachable by the
    activation recipe with each approximate reciprocal within one ulp; with
    correctly rounded reciprocals they are reproduced directly."""
    for fixture in vectors["vllm_scaled_fp4_quant"]["fixtures"]:
        x = np.tile(np.array(fixture["input"], dtype=np.float32), 4)[None, :]
        q = nvfp4.quantize_activations(x, fixture["global"])
        assert q.scales_linear[0, 0] == fixture["scale"]
        assert list(q.packed[0, :8]) == fixture["packed"]
        allowed_packed, allowed_scales = nvfp4.quantize_activations_candidates(x, fixture["global"])
        assert (allowed_scales[:, 0, 0] == fixture["scale"]).any()


def test_python_packer_vectors(vectors):
    p = vectors["python_packer"]
    codes = C.e2m1_encode(np.array(p["e2m1_input"], dtype=np.float32))
    assert C.pack_nibbles(codes).tobytes() == bytes.fromhex(p["e2m1_packed_hex"])
    assert list(C.e4m3_encode(np.array(p["e4m3_input"], dtype=np.float32))) == p["e4m3_codes"]
    # frozen group-16 recipe
    values = [2688., -2688.] + [0.] * 14
    values += p["e2m1_input"][:12] + [6., -6., .5, -.5]
    values += [0.] * 16 + [2 ** -16] + [0.] * 15
    w = nvfp4.pack_weights(np.array(values, dtype=np.float32).reshape(1, 64), 0.125)
    assert [w.weight_scale, w.input_scale] == p["group16_globals"]
    assert list(nvfp4.untile_scales(w.scales, 1, 64)[0]) == p["group16_scales"]
    assert w.data.tobytes() == bytes.fromhex("f7") + bytes(7) + bytes.fromhex(p["e2m1_packed_hex"]) + bytes(16)
    zero = nvfp4.pack_weights(np.array([0., -0.] * 32, dtype=np.float32).reshape(1, 64))
    assert zero.weight_scale == 1.0 and set(zero.data.reshape(-1)) == {p["zero_tensor_fp4_byte"]}
    f = fp8.pack_weights(np.array(p["fp8_tensor_input"], dtype=np.float32).reshape(1, 4), 0.125)
    assert f.weight_scale == 1.0 and list(f.data[0]) == p["fp8_tensor_codes"]


def test_e4m3_exhaustive():
    mags = C.E4M3_MAGNITUDES[:127]
    assert np.array_equal(C.e4m3_encode(mags), np.arange(127, dtype=np.uint8))
    mids = (mags[:-1] + mags[1:]) / 2
    assert list(C.e4m3_encode(mids)) == [i + (i % 2) for i in range(126)]
    assert np.array_equal(C.e4m3_encode(-mags[1:]), np.arange(1, 127, dtype=np.uint8) | 0x80)


def test_codecs_match_reference_python(packers):
    x = packers["codec_inputs"]
    assert np.array_equal(C.e4m3_encode(x), packers["e4m3_codes_scale1"])
    scaled = (np.abs(x) / np.float32(0.0737)).astype(np.float32)
    expect = packers["e4m3_codes_scale0737"]
    got = (C.e4m3_encode(scaled) & 0x7F) | (np.signbit(x).astype(np.uint8) << 7)
    assert np.array_equal(got, expect)
    assert np.array_equal(C.pack_nibbles(C.e2m1_encode(x)), packers["e2m1_packed"])
    assert np.array_equal(C.e4m3_decode(packers["e4m3_all_codes"]), packers["e4m3_all_decoded"])
    assert np.array_equal(C.bf16_bits(packers["bf16_bytes_inputs"]), packers["bf16_bytes_words"])


@pytest.mark.parametrize("name", ["normal", "wide_range", "sparse"])
def test_weight_packer_matches_reference_python(packers, name):
    values = packers[f"nvfp4_{name}_input"]
    w = nvfp4.pack_weights(values, 0.125)
    rows, columns = values.shape
    assert np.float32(w.weight_scale) == packers[f"nvfp4_{name}_globals"][0]
    assert np.array_equal(nvfp4.untile_scales(w.scales, rows, columns), packers[f"nvfp4_{name}_scales_linear"])
    assert np.array_equal(w.data, packers[f"nvfp4_{name}_packed"])
    assert np.array_equal(w.scales, packers[f"nvfp4_{name}_scales_swizzled"])
    assert w.scales.size == nvfp4.scale_storage_bytes(rows, columns)
    assert np.array_equal(nvfp4.dequantize(w), packers[f"nvfp4_{name}_dequantized"])
    f = fp8.pack_weights(values, 0.125)
    assert np.float32(f.weight_scale) == packers[f"fp8_{name}_scale"][0]
    assert np.array_equal(f.data, packers[f"fp8_{name}_codes"])


def test_layout_sizes(vectors):
    rows, width, total = vectors["layout"]["expert_entry_bytes"]
    assert rows * width // 2 + nvfp4.scale_storage_bytes(rows, width) + 8 == total
    # scale_offset is a bijection onto the storage of a full tile grid
    r, b = np.meshgrid(np.arange(256), np.arange(256 // 16), indexing="ij")
    offsets = nvfp4.scale_offset(r, b, 256).reshape(-1)
    assert np.array_equal(np.sort(offsets), np.arange(nvfp4.scale_storage_bytes(256, 256)))
