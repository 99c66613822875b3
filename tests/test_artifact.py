"""CPU tests of the artifact-container reader (gw_artifact_*: ArtifactFile::Open / ValidateMetadata / VerifyFull,
src/models/gemma4/26b_a4b/artifact.cc:105-221) on a file written by the reference's OWN writer and accepted by the
reference's own reader (tests/golden/make_artifact_golden.py): a six-tensor inventory with BF16, NVFP4 (rows padded
200 -> 256 and 704 -> 768) and FP8 entries.  Host code: no GPU."""
import ctypes
import hashlib
import json
import struct

import pytest

from gewell_b200 import _lib


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


@pytest.fixture(scope="module")
def description(golden_dir):
    return json.loads((golden_dir / "small_mixed.json").read_text())


def inventory_of(description):
    tensors = description["tensors"]
    array = (_lib.ArtifactTensorSpec * len(tensors))()
    for spec, t in zip(array, tensors):
        spec.layer, spec.role, spec.rank = t["layer"], t["role"], t["rank"]
        spec.rows, spec.columns, spec.projection = t["rows"], t["columns"], t["projection"]
    return array


def open_artifact(lib, path, inventory):
    handle = ctypes.c_void_p()
    status = lib.gw_artifact_open(str(path).encode(), inventory, len(inventory), ctypes.byref(handle))
    return status, handle, lib.gw_last_error().decode()


def test_reference_written_artifact_opens_and_verifies(lib, description, golden_dir):
    inventory = inventory_of(description)
    status, handle, message = open_artifact(lib, golden_dir / "small_mixed.gwt", inventory)
    assert status == _lib.GW_OK, message
    try:
        assert lib.gw_artifact_is_mixed(handle) == 1
        assert lib.gw_artifact_count(handle) == len(description["tensors"])
        assert lib.gw_artifact_file_bytes(handle) == description["file_bytes"]
        raw = (golden_dir / "small_mixed.gwt").read_bytes()
        for i, t in enumerate(description["tensors"]):
            entry = _lib.ArtifactEntry()
            assert lib.gw_artifact_entry_at(handle, i, ctypes.byref(entry)) == _lib.GW_OK
            assert (entry.offset, entry.bytes, entry.storage) == (t["offset"], t["bytes"], t["storage"])
            assert bytes(entry.sha256).hex() == t["sha256"]
            payload = ctypes.string_at(entry.data, entry.bytes)
            assert payload == raw[t["offset"]:t["offset"] + t["bytes"]]
            assert hashlib.sha256(payload).hexdigest() == t["sha256"]
            if t["storage"] != _lib.STORAGE_BF16:
                # the entry's byte count and content pass the per-entry checks, and bind to device addresses
                assert lib.gw_projection_entry_bytes(t["storage"], t["rows"], t["columns"]) == t["bytes"]
                assert lib.gw_validate_projection_entry(t["storage"], t["rows"], t["columns"], entry.data, entry.bytes) == _lib.GW_OK
                projection = _lib.Projection()
                device_base = 0x7000_0000_0000 + t["offset"]
                assert lib.gw_bind_projection(t["storage"], t["rows"], t["columns"], entry.data, device_base, entry.bytes,
                                              ctypes.byref(projection)) == _lib.GW_OK
                weight_scale, input_scale = struct.unpack("<ff", payload[-8:])
                if t["storage"] == _lib.STORAGE_NVFP4_W4A4:
                    padded = (t["rows"] + 127) // 128 * 128
                    assert projection.physical_output == padded and projection.output == t["rows"]
                    assert projection.nvfp4_scales == device_base + padded * t["columns"] // 2
                    assert (projection.nvfp4_weight_scale, projection.nvfp4_input_scale) == (weight_scale, input_scale)
                else:
                    assert projection.fp8_data == device_base
                    assert (projection.fp8_weight_scale, projection.fp8_input_scale) == (weight_scale, input_scale)
        assert lib.gw_artifact_entry_at(handle, len(description["tensors"]), ctypes.byref(_lib.ArtifactEntry())) == _lib.GW_INVALID_ARGUMENT
        assert lib.gw_artifact_verify_full(handle) == _lib.GW_OK, lib.gw_last_error().decode()
    finally:
        lib.gw_artifact_close(handle)


def rewrite_header_hash(raw: bytearray):
    raw[296:328] = bytes(32)
    raw[296:328] = hashlib.sha256(bytes(raw[:4096])).digest()


@pytest.mark.parametrize("case,expected", [
    ("magic", "wrong 26B artifact identity"),
    ("geometry", "invalid 26B header geometry"),
    ("alias", "invalid 26B tied-head alias"),
    ("reserved", "nonzero 26B header reserved bytes"),
    ("header_hash", "26B header checksum mismatch"),
    ("table_hash", "26B entry table checksum mismatch"),
    ("entry_shape", "invalid 26B tensor entry 2"),
    ("size", "invalid 26B artifact size"),
    ("globals", "invalid 26B global scales"),
    ("truncated", "truncated 26B artifact"),
    ("not_projection", "quantized 26B tensor is not a projection"),
])
def test_metadata_rejections(lib, description, golden_dir, tmp_path, case, expected):
    raw = bytearray((golden_dir / "small_mixed.gwt").read_bytes())
    inventory = inventory_of(description)
    tensors = description["tensors"]
    if case == "magic":
        raw[:8] = b"G4A4XXXX"
    elif case == "geometry":
        raw[8 + 4 * 3:8 + 4 * 4] = struct.pack("<I", len(tensors) + 1); rewrite_header_hash(raw)
    elif case == "alias":
        raw[92:96] = struct.pack("<I", 1); rewrite_header_hash(raw)
    elif case == "reserved":
        raw[100] = 1; rewrite_header_hash(raw)
    elif case == "header_hash":
        raw[170] ^= 1                                   # a digest field changes, the header's own digest does not
    elif case == "table_hash":
        raw[4096 + 40] ^= 1                             # an entry's stored SHA changes: the table digest no longer matches
    elif case == "entry_shape":
        inventory[2].rows = 201                         # the file says 200
    elif case == "size":
        raw += bytes(4096)
    elif case == "globals":
        t = tensors[2]
        raw[t["offset"] + t["bytes"] - 4:t["offset"] + t["bytes"]] = struct.pack("<f", 0.0)
    elif case == "truncated":
        raw = raw[:6000]
    elif case == "not_projection":
        inventory[2].projection = 0
    path = tmp_path / "artifact.gwt"
    path.write_bytes(bytes(raw))
    status, handle, message = open_artifact(lib, path, inventory)
    if status == _lib.GW_OK:
        lib.gw_artifact_close(handle)
    assert status == _lib.GW_INVALID_ARGUMENT and message == expected


@pytest.mark.parametrize("case,expected", [
    ("payload_byte", "26B tensor checksum mismatch"),
    ("tensor_padding", "nonzero 26B tensor padding"),
    ("table_padding", "nonzero 26B table padding"),
    ("weight_padding", "nonzero 26B NVFP4 weight padding"),
    ("payload_hash", "26B payload checksum mismatch"),
])
def test_full_verification_rejections(lib, description, golden_dir, tmp_path, case, expected):
    raw = bytearray((golden_dir / "small_mixed.gwt").read_bytes())
    tensors = description["tensors"]
    if case == "payload_byte":
        raw[tensors[0]["offset"] + 3] ^= 0x10
    elif case == "tensor_padding":
        raw[tensors[1]["offset"] + tensors[1]["bytes"] + 5] = 7
    elif case == "table_padding":
        raw[4096 + 72 * len(tensors) + 9] = 1
    elif case == "weight_padding":
        t = tensors[2]                                  # rows 200..255 of the packed matrix are padding
        raw[t["offset"] + 200 * t["columns"] // 2 + 1] = 0x11
    elif case == "payload_hash":
        raw[264] ^= 1; rewrite_header_hash(raw)
    path = tmp_path / "artifact.gwt"
    path.write_bytes(bytes(raw))
    status, handle, message = open_artifact(lib, path, inventory_of(description))
    assert status == _lib.GW_OK, message               # the metadata is intact
    try:
        assert lib.gw_artifact_verify_full(handle) == _lib.GW_INVALID_ARGUMENT
        assert lib.gw_last_error().decode() == expected
    finally:
        lib.gw_artifact_close(handle)
