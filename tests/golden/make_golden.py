#!/usr/bin/env python3
"""Generate packer / swizzle / dequantiser fixtures from the reference's own
importable Python code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/gewell

It imports tools/convert.py (quantize_e4m3, quantize_e2m1,
quantize_nvfp4_tensor, quantize_tensor), tools/nvfp4_artifact.py
(swizzle_scale_chunk) and tools/safetensors_source.py (decode_e4m3, bf16_bytes)
from that checkout, feeds them seeded inputs and stores inputs and outputs in
tests/golden/reference_packers.npz.  The fixture travels with the repository;
the reference does not need to be present when the tests run.
"""

import argparse
import sys
import tempfile
from pathlib import Path

import numpy as np


def bf16_words(values):
    """Truncate FP32 to BF16 words the way the reference's test helper does
    (tests/test_mixed_conversion.py:18-22); inputs are made BF16-exact first."""
    return (np.asarray(values, dtype=np.float32).view(np.uint32) >> 16).astype("<u2")


def to_bf16_exact(values):
    bits = np.asarray(values, dtype=np.float32).view(np.uint32)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32)


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", type=Path, required=True)
    parser.add_argument("--output", type=Path,
                        default=Path(__file__).with_name("reference_packers.npz"))
    args = parser.parse_args()
    sys.path.insert(0, str(args.reference))
    sys.dont_write_bytecode = True
    from tools import bf16_artifact as bf16
    from tools import convert, nvfp4_artifact as native, safetensors_source as source

    rng = np.random.default_rng(20261125)
    out = {}

    # --- scalar codecs on awkward values -----------------------------------
    grid = np.concatenate([
        rng.normal(0, 1, 4096), rng.normal(0, 100, 2048), rng.uniform(-8, 8, 4096),
        convert.E4M3_VALUES, -convert.E4M3_VALUES,
        (convert.E4M3_VALUES[:-1] + convert.E4M3_VALUES[1:]) / 2,
        [0.0, -0.0, 448, 449, 464, 1e6, -1e6, 2.0 ** -10, 3 * 2.0 ** -10, 2.0 ** -9],
        np.arange(-7, 7.01, 0.125)]).astype(np.float32)
    if grid.size % 2:
        grid = grid[:-1]
    out["codec_inputs"] = grid
    out["e4m3_codes_scale1"] = np.frombuffer(convert.quantize_e4m3(grid, 1.0), dtype=np.uint8)
    out["e4m3_codes_scale0737"] = np.frombuffer(convert.quantize_e4m3(grid, 0.0737), dtype=np.uint8)
    out["e2m1_packed"] = np.frombuffer(convert.quantize_e2m1(grid), dtype=np.uint8)
    all_codes = bytes(c for c in range(256) if c & 0x7F != 0x7F)
    out["e4m3_all_codes"] = np.frombuffer(all_codes, dtype=np.uint8)
    out["e4m3_all_decoded"] = source.decode_e4m3(all_codes)
    out["bf16_bytes_inputs"] = grid
    out["bf16_bytes_words"] = np.frombuffer(source.bf16_bytes(grid), dtype="<u2")

    # --- whole-tensor packers -------------------------------------------------
    with tempfile.TemporaryDirectory() as temporary:
        root = Path(temporary)
        cases = {
            "normal": to_bf16_exact(rng.normal(0, 0.02, (256, 192))),
            "wide_range": to_bf16_exact(rng.normal(0, 1, (128, 128)) * np.exp2(rng.integers(-14, 6, (128, 1)))),
            "sparse": to_bf16_exact(np.where(rng.random((128, 64)) < 0.6, 0, rng.normal(0, 3, (128, 64)))),
        }
        for name, values in cases.items():
            words = bf16_words(values)
            path = root / f"{name}.bf16"
            path.write_bytes(words.tobytes())
            tensor = bf16.SourceTensor(path, path.name, name, 0, words.nbytes)
            packed = convert.quantize_nvfp4_tensor(tensor, root / f"{name}.fp4", 0.125)
            weight_scale, input_scale = native.validate_globals(packed.globals)
            rows, columns = values.shape
            linear = packed.block_scales.path.read_bytes()
            swizzled = b"".join(
                native.swizzle_scale_chunk(linear[r * (columns // 16):min(rows, r + 128) * (columns // 16)],
                                           min(128, rows - r), columns // 16)
                for r in range(0, rows, 128))
            out[f"nvfp4_{name}_input"] = values
            out[f"nvfp4_{name}_packed"] = np.frombuffer(packed.weight.path.read_bytes(), dtype=np.uint8).reshape(rows, columns // 2)
            out[f"nvfp4_{name}_scales_linear"] = np.frombuffer(linear, dtype=np.uint8).reshape(rows, columns // 16)
            out[f"nvfp4_{name}_scales_swizzled"] = np.frombuffer(swizzled, dtype=np.uint8)
            out[f"nvfp4_{name}_globals"] = np.array([weight_scale, input_scale], dtype=np.float32)
            # the reference's CPU dequantiser (materialize_bf16) on its own packing
            weight = source.Weight(packed.weight, "U8", values.shape, packed.block_scales,
                                   weight_scale, input_scale)
            restored = source.materialize_bf16(weight, root / f"{name}.restored")
            out[f"nvfp4_{name}_dequantized"] = np.frombuffer(restored.path.read_bytes(), dtype="<u2").reshape(rows, columns)

            fp8_packed = convert.quantize_tensor(tensor, root / f"{name}.fp8", 0.125)
            fp8_scale, _ = native.validate_globals(fp8_packed.globals)
            out[f"fp8_{name}_codes"] = np.frombuffer(fp8_packed.weight.path.read_bytes(), dtype=np.uint8).reshape(rows, columns)
            out[f"fp8_{name}_scale"] = np.array([fp8_scale], dtype=np.float32)

    np.savez_compressed(args.output, **out)
    print(f"wrote {args.output} ({args.output.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main()
