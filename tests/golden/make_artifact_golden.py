#!/usr/bin/env python3
"""Write a small 26B-A4B mixed artifact (G4A4MIX1) with the reference's OWN writer and packers.

Run where the reference checkout is available:

    python tests/golden/make_artifact_golden.py --reference /path/to/gewell

The reference's writer (tools/gemma4_26b_mixed_artifact.py: write_artifact) takes the model's tensor inventory
from tools/gemma4_26b_contract.native_tensor_specs(); this script substitutes a six-tensor inventory of the same
TensorSpec type (an embedding, a norm vector, an NVFP4 projection whose 200 rows pad to 256, an FP8 projection, an
NVFP4 expert projection of the real 704-row shape, a final norm), feeds the writer tensors packed by the reference's
quantize_nvfp4_tensor / quantize_tensor, lets the reference's own read_metadata accept the file, and stores

    tests/golden/small_mixed.gwt         the artifact, byte for byte as the reference wrote it
    tests/golden/small_mixed.json        the inventory and, per entry, storage type, offset, byte count, SHA-256

The fixture travels with the repository; the reference does not need to be present when the tests run.
"""

import argparse
import hashlib
import json
import sys
import tempfile
from pathlib import Path

import numpy as np


def bf16_words(values):
    bits = np.asarray(values, dtype=np.float32).view(np.uint32)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16
    return rounded.astype("<u2")


def main():
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--reference", type=Path, required=True)
    parser.add_argument("--output", type=Path, default=Path(__file__).with_name("small_mixed.gwt"))
    args = parser.parse_args()
    sys.path.insert(0, str(args.reference))
    sys.dont_write_bytecode = True
    from tools import bf16_artifact as wire
    from tools import convert, nvfp4_artifact as native
    from tools import gemma4_26b_contract as contract
    from tools import gemma4_26b_mixed_artifact as mixed
    from tools.gemma4_26b_quantization import StorageType, TARGET_ROLES

    Role, Spec = contract.Role, contract.TensorSpec
    prefix = "model.language_model."
    inventory = [
        (Spec(0, Role.EMBEDDING, -1, -1, (16, 32), prefix + "embed_tokens.weight"), StorageType.BF16),
        (Spec(1, Role.INPUT_NORM, 0, -1, (64,), prefix + "layers.0.input_layernorm.weight"), StorageType.BF16),
        (Spec(2, Role.GATE_PROJ, 0, -1, (200, 128), prefix + "layers.0.mlp.gate_proj.weight"), StorageType.NVFP4_W4A4),
        (Spec(3, Role.DOWN_PROJ, 0, -1, (48, 64), prefix + "layers.0.mlp.down_proj.weight"), StorageType.FP8_W8A8),
        (Spec(4, Role.EXPERT_GATE_PROJ, 0, 3, (704, 64), prefix + "layers.0.experts.gate_up_proj"), StorageType.NVFP4_W4A4),
        (Spec(5, Role.FINAL_NORM, -1, -1, (64,), prefix + "norm.weight"), StorageType.BF16),
    ]
    specs = [spec for spec, _ in inventory]
    mixed.native_tensor_specs = lambda: specs           # the writer and the reader look the inventory up here

    rng = np.random.default_rng(20261126)
    with tempfile.TemporaryDirectory() as temporary:
        root = Path(temporary)
        sources = []
        for spec, storage in inventory:
            values = rng.normal(0, 0.05, spec.shape).astype(np.float32)
            words = bf16_words(values)
            path = root / f"{spec.physical_id}.bf16"
            path.write_bytes(words.tobytes())
            source_name = spec.separate_source_name if spec.expert >= 0 else spec.source_name
            tensor = wire.SourceTensor(path, path.name, source_name, 0, words.nbytes)
            if storage == StorageType.BF16:
                sources.append(native.TensorSource(tensor, storage))
            elif storage == StorageType.NVFP4_W4A4:
                sources.append(convert.quantize_nvfp4_tensor(tensor, root / f"{spec.physical_id}.fp4", 0.0625))
            else:
                sources.append(convert.quantize_tensor(tensor, root / f"{spec.physical_id}.fp8", 0.03125))
        if args.output.exists():
            args.output.unlink()
        config_hash, index_hash = hashlib.sha256(b"config").digest(), hashlib.sha256(b"index").digest()
        sizes = mixed.write_artifact(args.output, sources, config_hash, index_hash)
        header, entries = mixed.read_metadata(args.output)          # the reference's own reader accepts the file

    description = {
        "format": sizes["format"], "file_bytes": sizes["file_bytes"], "data_offset": sizes["data_offset"],
        "tensors": [{"layer": spec.layer, "role": int(spec.role), "rank": len(spec.shape), "rows": spec.shape[0],
                     "columns": spec.shape[1] if len(spec.shape) == 2 else 0, "projection": int(spec.role in TARGET_ROLES),
                     "storage": int(entry.storage_type), "offset": entry.file_offset, "bytes": entry.byte_length,
                     "sha256": entry.sha256.hex()} for spec, entry in zip(specs, entries)],
    }
    args.output.with_suffix(".json").write_text(json.dumps(description, indent=1) + "\n")
    print(f"wrote {args.output} ({args.output.stat().st_size} bytes) and {args.output.with_suffix('.json').name}")


if __name__ == "__main__":
    main()
