"""Safetensors weight sources (host logic, no device): the reference's own unit tests of
crates/forja-host/src/weights.rs:535-830 restated against the C ABI, plus JSON corner cases of the
header reader."""
import json
import os
import struct

import pytest

import forja_b200 as fb
from forja_b200 import weights as W


def write_file(path, header: str, data: bytes, pad: bool = True):
    raw = header.encode("utf-8")
    if pad:
        while (len(raw) + 8) % 8:
            raw += b" "
    path.write_bytes(struct.pack("<Q", len(raw)) + raw + data)
    return path


def open_source(tmp_path, header, data, pad=True):
    return W.Safetensors.open(write_file(tmp_path / "model.bin", header, data, pad))


def entry(dtype, shape, lo, hi):
    return {"dtype": dtype, "shape": shape, "data_offsets": [lo, hi]}


def test_parses_supported_tensor_metadata(tmp_path):
    header = json.dumps({"a": entry("F32", [1], 0, 4), "b": entry("BF16", [2], 4, 8), "c": entry("U32", [1], 8, 12)}, separators=(",", ":"))
    source = open_source(tmp_path, header, bytes(12))
    tensors = source.tensors()
    assert len(tensors) == 3
    assert tensors[0].name == "a" and tensors[0].dtype == fb.F32
    assert tensors[1].shape == (2,) and tensors[1].dtype == fb.BF16
    assert tensors[2].dtype == fb.U32 and tensors[2].byte_offset == 8 and tensors[2].byte_len == 4
    assert source.shard_name is None and source.file_len == 8 + source.data_start - 8 + 12


def test_tensors_are_ordered_by_offset_and_metadata_is_skipped(tmp_path):
    header = json.dumps({"__metadata__": {"format": "pt"}, "late": entry("F16", [2, 2], 8, 16), "early": entry("F32", [2], 0, 8)})
    names = [t.name for t in open_source(tmp_path, header, bytes(16)).tensors()]
    assert names == ["early", "late"]


@pytest.mark.parametrize("header,data,kind", [
    ({"a": entry("F32", [2], 0, 8)}, bytes(4), "Truncated"),                                              # rejects_truncated_tensor_data
    ({"a": entry("F32", [2], 0, 8), "b": entry("F32", [1], 4, 8)}, bytes(8), "OverlappingRanges"),         # rejects_overlapping_ranges
    ({"a": entry("F16", [4], 0, 8)}, bytes(6), "Truncated"),                                              # rejects_ranges_past_the_file_end
    ({"a": entry("F8_E4M3", [1], 0, 1)}, bytes(1), "UnsupportedDtype"),                                    # rejects_unknown_dtypes
    ({"a": entry("F32", [3], 0, 8)}, bytes(8), "InvalidRange"),                                            # byte range != shape x element size
    ({"a": entry("F32", [1], 8, 4)}, bytes(8), "InvalidRange"),                                            # end before start
    ({"a": entry("F32", [4294967295, 4294967295, 4294967295], 0, 4)}, bytes(4), "InvalidRange"),           # element count overflows
    ({"a": entry("F32", [4294967296], 0, 4)}, bytes(4), "InvalidHeader"),                                  # extent is not a u32
    ({"a": entry("F32", [-1], 0, 4)}, bytes(4), "InvalidHeader"),
    ({"a": entry("F32", [1.5], 0, 4)}, bytes(4), "InvalidHeader"),
    ({"a": {"dtype": "F32", "shape": [1]}}, bytes(4), "InvalidHeader"),                                    # data_offsets missing
    ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4, 8]}}, bytes(8), "InvalidHeader"),
    ({"a": {"shape": [1], "data_offsets": [0, 4]}}, bytes(4), "InvalidHeader"),
    ({"a": 7}, bytes(4), "InvalidHeader"),
])
def test_rejects_invalid_headers(tmp_path, header, data, kind):
    with pytest.raises(W.WeightError) as e:
        open_source(tmp_path, json.dumps(header), data)
    assert e.value.kind == kind
    if kind == "UnsupportedDtype":
        assert e.value.message == "F8_E4M3"


def test_rejects_duplicate_tensor_names(tmp_path):
    one = json.dumps(entry("F32", [1], 0, 4))
    with pytest.raises(W.WeightError) as e:
        open_source(tmp_path, '{"a":%s,"a":%s}' % (one, one), bytes(4))
    assert e.value.kind == "InvalidHeader" and "duplicate" in e.value.message


def test_rejects_deeply_nested_headers(tmp_path):
    with pytest.raises(W.WeightError) as e:
        open_source(tmp_path, '{"a":%s0%s}' % ("[" * 256, "]" * 256), b"")
    assert e.value.kind == "InvalidHeader"
    # 100 levels are fine for the reader (and then fail the schema check, not the depth check)
    with pytest.raises(W.WeightError) as e:
        open_source(tmp_path, '{"a":%s0%s}' % ("[" * 100, "]" * 100), b"")
    assert "not an object" in e.value.message


def test_rejects_headers_over_the_size_cap_before_reading_them(tmp_path):
    path = tmp_path / "cap.bin"
    path.write_bytes(struct.pack("<Q", 100 * 1024 * 1024 + 1))
    with pytest.raises(W.WeightError) as e:
        W.Safetensors.open(path)
    assert e.value.kind == "HeaderTooLarge"


def test_unpadded_header_and_data_region(tmp_path):
    # aligns_tensor_offsets_to_the_data_region
    header = '{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
    source = open_source(tmp_path, header, bytes(4), pad=False)
    assert source.tensors()[0].is_dtype_aligned
    assert source.data_start == 8 + len(header) and source.file_len == source.data_start + 4


def test_rejects_truncated_prefix_header_and_malformed_json(tmp_path):
    (tmp_path / "short").write_bytes(b"\x01\x02")
    with pytest.raises(W.WeightError) as e:
        W.Safetensors.open(tmp_path / "short")
    assert e.value.kind == "Truncated"
    (tmp_path / "cut").write_bytes(struct.pack("<Q", 50) + b"{}")
    with pytest.raises(W.WeightError) as e:
        W.Safetensors.open(tmp_path / "cut")
    assert e.value.kind == "Truncated"
    for text in ("{", '{"a":}', '{"a":1,}', '{"a":01}', '{"a":"\\x"}', '{"a":1} x', "[]", '{"a":"\\ud800"}', '{"a":tru}'):
        with pytest.raises(W.WeightError) as e:
            open_source(tmp_path, text, b"")
        assert e.value.kind == "InvalidHeader", text
    with pytest.raises(W.WeightError) as e:
        W.Safetensors.open(tmp_path / "missing")
    assert e.value.kind == "Io"
    with pytest.raises(W.WeightError) as e:
        W.Safetensors.open(tmp_path)
    assert e.value.kind == "NotRegularFile"


def test_escaped_names_are_decoded(tmp_path):
    header = '{"caf\\u00e9 \\ud83d\\ude00\\n":{"dtype":"F32","shape":[],"data_offsets":[0,4]}}'
    assert open_source(tmp_path, header, bytes(4)).tensors()[0].name == "café \U0001F600\n"


SHARD_A = '{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'
SHARD_B = '{"b":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}'


def write_index(directory, contents):
    path = directory / "model.safetensors.index.json"
    path.write_bytes(contents if isinstance(contents, bytes) else contents.encode("utf-8"))
    return path


def invalid_index(directory, contents):
    with pytest.raises(W.WeightError) as e:
        W.Safetensors.open_all(write_index(directory, contents))
    return e.value


def test_opens_validated_shard_indexes(tmp_path):
    write_file(tmp_path / "first.safetensors", SHARD_A, bytes(4))
    write_file(tmp_path / "second.safetensors", SHARD_B, bytes(4))
    index = write_index(tmp_path, '{"metadata":{"total_size":8},"weight_map":{"b":"second.safetensors","a":"first.safetensors"}}')
    sources = W.Safetensors.open_all(index)
    assert len(sources) == 2
    assert sources[0].tensors()[0].name == "a" and sources[0].shard_name == "first.safetensors"
    assert sources[1].tensors()[0].name == "b" and sources[1].shard_name == "second.safetensors"
    # a path that is not an index opens as one file
    assert len(W.Safetensors.open_all(tmp_path / "first.safetensors")) == 1


@pytest.mark.parametrize("contents", [
    '{"weight_map":{"a":"../x.safetensors"}}',        # rejects_parent_shard_paths
    '{"weight_map":{"a":"/tmp/absolute.safetensors"}}',  # rejects_absolute_shard_paths
    '{"weight_map":{"a":"nested/x.safetensors"}}',    # rejects_shard_names_with_embedded_separators
    '{"weight_map":{"a":"nested\\\\x.safetensors"}}',
    '{"weight_map":{"a":"shard.bin"}}',               # rejects_non_safetensors_shards
    '{"weight_map":{}}',                              # rejects_empty_weight_maps
    '{"weight_map":{"a":7}}',                         # rejects_non_string_shard_values
    '{',                                              # rejects_malformed_indexes
    '{"metadata":{}}',                                # weight_map missing
    '{"weight_map":{"a":"s.safetensors","a":"s.safetensors"}}',
])
def test_rejects_invalid_indexes(tmp_path, contents):
    assert invalid_index(tmp_path, contents).kind == "InvalidIndex"


def test_rejects_shards_that_do_not_match_the_weight_map(tmp_path):
    write_file(tmp_path / "shard.safetensors", SHARD_B, bytes(4))
    assert invalid_index(tmp_path, '{"weight_map":{"a":"shard.safetensors"}}').kind == "InvalidIndex"  # rejects_shards_missing_declared_tensors
    two = '{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"b":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}'
    write_file(tmp_path / "shard.safetensors", two, bytes(8))
    assert invalid_index(tmp_path, '{"weight_map":{"a":"shard.safetensors"}}').kind == "InvalidIndex"  # rejects_shards_with_undeclared_tensors


def test_rejects_indexes_over_the_size_cap(tmp_path):
    index = write_index(tmp_path, b"")
    with open(index, "r+b") as f:
        f.truncate(100 * 1024 * 1024 + 1)
    with pytest.raises(W.WeightError) as e:
        W.Safetensors.open_all(index)
    assert e.value.kind == "InvalidIndex"


def test_rejects_too_many_shards(tmp_path):
    weight_map = {f"tensor-{i}": f"shard-{i}.safetensors" for i in range(1025)}
    assert invalid_index(tmp_path, json.dumps({"weight_map": weight_map})).kind == "InvalidIndex"


def test_rejects_shards_symlinked_outside_the_model_directory(tmp_path):
    model = tmp_path / "model"
    model.mkdir()
    outside = write_file(tmp_path / "outside.safetensors", SHARD_A, bytes(4))
    os.symlink(outside, model / "shard.safetensors")
    assert invalid_index(model, '{"weight_map":{"a":"shard.safetensors"}}').kind == "InvalidIndex"


def test_rejects_fifo_shards_without_opening_them(tmp_path):
    os.mkfifo(tmp_path / "shard.safetensors")
    assert invalid_index(tmp_path, '{"weight_map":{"a":"shard.safetensors"}}').kind == "NotRegularFile"
