"""The safetensors weight store and the Q4 matrix descriptor (host side, no GPU).

The first block restates the reference's own format tests (src/model.rs:717-860 for the store,
src/native.rs:5730-5755 for the matrix layout) against `MlxWeightStore` / `Q4AffineMatrix`; the rest covers
what those tests leave out: header limits, offset ranges, multi-shard projections, arbitrary header padding.
"""
import json
import os
import struct

import numpy as np
import pytest

UP = "language_model.model.layers.0.mlp.up_proj"


@pytest.fixture(scope="module")
def W():
    from qwen38_metal_b200 import build, weights

    build.build()
    return weights


def fixture_config(directory):
    """write_fixture_config, src/model.rs:879-900"""
    with open(os.path.join(directory, "config.json"), "w") as f:
        f.write("""{
          "architectures": ["Qwen3_5ForConditionalGeneration"],
          "model_type": "qwen3_5",
          "quantization_config": {"bits": 4, "group_size": 64, "mode": "affine"},
          "text_config": {"model_type": "qwen3_5_text", "hidden_size": 5120, "num_hidden_layers": 4,
            "num_key_value_heads": 4, "head_dim": 256,
            "layer_types": ["linear_attention", "linear_attention", "linear_attention", "full_attention"],
            "mtp_num_hidden_layers": 1}
        }""")


def fixture_index(directory, weight_map):
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": weight_map}, f)


def raw_shard(path, header: dict, data: bytes, header_bytes=None):
    blob = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob) if header_bytes is None else header_bytes))
        f.write(blob)
        f.write(data)


def fixture_shard(path, names=(UP + ".weight", UP + ".scales", UP + ".biases")):
    """write_fixture_shard_with_names, src/model.rs:920-950: U8 [4] + F16 [2] + F16 [2], twelve zero bytes"""
    raw_shard(path, {
        names[0]: {"dtype": "U8", "shape": [4], "data_offsets": [0, 4]},
        names[1]: {"dtype": "F16", "shape": [2], "data_offsets": [4, 8]},
        names[2]: {"dtype": "F16", "shape": [2], "data_offsets": [8, 12]},
    }, bytes(12))


def full_map():
    return {UP + ".weight": "model.safetensors", UP + ".scales": "model.safetensors", UP + ".biases": "model.safetensors"}


def kind_of(err):
    return err.value.kind


# ---- the reference's tests ---------------------------------------------------------------------------

def test_maps_safetensors_tensor_ranges(W, tmp_path):
    """maps_safetensors_tensor_ranges_without_copying_them_to_the_heap, src/model.rs:792-817, plus the counts of
    reads_an_mlx_affine_manifest_without_loading_tensor_data, :720-747"""
    d = str(tmp_path)
    fixture_config(d)
    fixture_index(d, full_map())
    fixture_shard(os.path.join(d, "model.safetensors"))
    store = W.MlxWeightStore(d)
    tensor = store.tensor(UP + ".weight")
    assert store.shard_count() == 1
    assert store.tensor_count() == 3
    assert tensor.dtype == "U8"
    assert tensor.shape == (4,)
    assert store.tensor_data(UP + ".weight") == bytes(4)
    assert store.mapped_bytes() > tensor.byte_len
    assert store.indexed_tensor_bytes() == 12
    assert store.quantized_tensor_groups() == 1
    assert store.tensor("absent") is None and store.tensor_data("absent") is None
    store.close()


def test_rejects_a_quantized_weight_with_a_missing_affine_companion(W, tmp_path):
    """src/model.rs:819-843"""
    from qwen38_metal_b200 import Q4RuntimeError

    d = str(tmp_path)
    fixture_config(d)
    fixture_index(d, {UP + ".weight": "model.safetensors", UP + ".scales": "model.safetensors"})
    fixture_shard(os.path.join(d, "model.safetensors"))
    with pytest.raises(Q4RuntimeError) as err:
        W.MlxWeightStore(d)
    assert kind_of(err) == "IncompleteAffineGroup" and "biases" in str(err.value)


def test_rejects_an_index_that_tries_to_escape_the_model_directory(W, tmp_path):
    """src/model.rs:845-860"""
    from qwen38_metal_b200 import Q4RuntimeError

    d = str(tmp_path)
    fixture_config(d)
    for bad in ("../outside.safetensors", "/etc/passwd", "a/../../b.safetensors", "./model.safetensors"):
        fixture_index(d, {UP + ".weight": bad})
        with pytest.raises(Q4RuntimeError) as err:
            W.MlxWeightStore(d)
        assert kind_of(err) == "UnsafeShardPath"


def mlx(dtype, shape, byte_len):
    from qwen38_metal_b200.weights import MlxTensor

    return MlxTensor(dtype, tuple(shape), 0, 0, byte_len)


def test_accepts_an_mlx_q4_affine_matrix_layout(W):
    """src/native.rs:5730-5743"""
    m = W.Q4AffineMatrix.from_tensors("layer.weight", mlx("U32", [3, 16], 192), mlx("BF16", [3, 2], 12), mlx("BF16", [3, 2], 12))
    assert m.input_elements == 128
    assert m.output_rows == 3


def test_rejects_a_wrong_scale_layout(W):
    """src/native.rs:5745-5757"""
    from qwen38_metal_b200 import Q4RuntimeError

    with pytest.raises(Q4RuntimeError) as err:
        W.Q4AffineMatrix.from_tensors("layer.weight", mlx("U32", [3, 16], 192), mlx("BF16", [3, 3], 18), mlx("BF16", [3, 2], 12))
    assert kind_of(err) == "InvalidAffineTensor"


# ---- beyond the reference's tests --------------------------------------------------------------------

@pytest.mark.parametrize("weight,scales,biases,kind", [
    (("F32", [3, 16], 192), ("BF16", [3, 2], 12), ("BF16", [3, 2], 12), "InvalidQuantizedWeight"),   # dtype
    (("U32", [3, 16, 1], 192), ("BF16", [3, 2], 12), ("BF16", [3, 2], 12), "InvalidQuantizedWeight"),  # rank
    (("U32", [3, 12], 144), ("BF16", [3, 1], 6), ("BF16", [3, 1], 6), "InvalidQuantizedWeight"),     # K=96 not grouped
    (("U32", [0, 16], 0), ("BF16", [0, 2], 0), ("BF16", [0, 2], 0), "InvalidQuantizedWeight"),       # no rows
    (("U32", [3, 16], 188), ("BF16", [3, 2], 12), ("BF16", [3, 2], 12), "TensorByteLength"),
    (("U32", [3, 16], 192), ("BF16", [3, 2], 10), ("BF16", [3, 2], 12), "TensorByteLength"),
    (("U32", [3, 16], 192), ("F16", [3, 2], 12), ("BF16", [3, 2], 12), "InvalidAffineTensor"),
    (("U32", [3, 16], 192), ("BF16", [3, 2], 12), ("BF16", [2, 2], 8), "InvalidAffineTensor"),
    (("U32", [1 << 62, 16], 192), ("BF16", [3, 2], 12), ("BF16", [3, 2], 12), "DimensionOverflow"),
])
def test_matrix_layout_rejections(W, weight, scales, biases, kind):
    from qwen38_metal_b200 import Q4RuntimeError

    with pytest.raises(Q4RuntimeError) as err:
        W.Q4AffineMatrix.from_tensors("layer.weight", mlx(*weight), mlx(*scales), mlx(*biases))
    assert kind_of(err) == kind


def test_header_length_limits(W, tmp_path):
    """read_safetensors_header, src/model.rs:345-372: files under 8 bytes, lengths past the file or past 128 MiB"""
    from qwen38_metal_b200 import Q4RuntimeError

    d = str(tmp_path)
    fixture_config(d)
    fixture_index(d, full_map())
    shard = os.path.join(d, "model.safetensors")
    for content in (b"\x01\x02\x03", struct.pack("<Q", 100) + b"{}", struct.pack("<Q", (128 << 20) + 1) + b"{}"):
        with open(shard, "wb") as f:
            f.write(content)
        with pytest.raises(Q4RuntimeError) as err:
            W.MlxWeightStore(d)
        assert kind_of(err) == "InvalidHeaderLength"


@pytest.mark.parametrize("entry,kind", [
    ({"dtype": "U8", "shape": [4], "data_offsets": [0, 13]}, "InvalidTensorOffsets"),   # past the data section
    ({"dtype": "U8", "shape": [4], "data_offsets": [8, 4]}, "InvalidTensorOffsets"),    # reversed
    ({"dtype": "", "shape": [4], "data_offsets": [0, 4]}, "InvalidTensorMetadata"),
    ({"dtype": "U8", "shape": [], "data_offsets": [0, 4]}, "InvalidTensorMetadata"),
    ({"dtype": "U8", "shape": [4]}, "Json"),
    ({"dtype": "U8", "shape": [4], "data_offsets": [0, -4]}, "Json"),
    ({"dtype": "U8", "shape": [4.5], "data_offsets": [0, 4]}, "Json"),
])
def test_bad_tensor_entries(W, tmp_path, entry, kind):
    from qwen38_metal_b200 import Q4RuntimeError

    d = str(tmp_path)
    fixture_config(d)
    fixture_index(d, {"t": "model.safetensors"})
    raw_shard(os.path.join(d, "model.safetensors"), {"t": entry, "__metadata__": {"format": "mlx"}}, bytes(12))
    with pytest.raises(Q4RuntimeError) as err:
        W.MlxWeightStore(d)
    assert kind_of(err) == kind


def test_missing_files_and_tensors(W, tmp_path):
    from qwen38_metal_b200 import Q4RuntimeError

    d = str(tmp_path)
    with pytest.raises(Q4RuntimeError) as err:
        W.MlxWeightStore(d)                      # no config.json
    assert kind_of(err) == "Read"
    fixture_config(d)
    with pytest.raises(Q4RuntimeError) as err:
        W.MlxWeightStore(d)                      # no index
    assert kind_of(err) == "Read"
    fixture_index(d, {"elsewhere": "model.safetensors"})
    with pytest.raises(Q4RuntimeError) as err:
        W.MlxWeightStore(d)                      # shard file absent
    assert kind_of(err) == "Read"
    fixture_shard(os.path.join(d, "model.safetensors"))
    with pytest.raises(Q4RuntimeError) as err:
        W.MlxWeightStore(d)                      # indexed tensor not in the shard header
    assert kind_of(err) == "MissingIndexedTensor"
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        f.write("{\"weight_map\": {\"a\": 3}}")
    with pytest.raises(Q4RuntimeError) as err:
        W.MlxWeightStore(d)
    assert kind_of(err) == "Json"


@pytest.mark.parametrize("config,kind", [
    ({"model_type": "qwen3_5"}, "MissingQuantization"),
    ({"quantization": {"bits": 8, "group_size": 64, "mode": "affine"}}, "UnsupportedQuantization"),
    ({"quantization_config": {"bits": 4, "group_size": 0, "mode": "affine"}}, "UnsupportedQuantization"),
    ({"quantization_config": {"bits": 4, "group_size": 64, "mode": "mxfp4"}}, "UnsupportedQuantization"),
])
def test_quantization_block_is_checked(W, tmp_path, config, kind):
    """src/model.rs:229-240"""
    from qwen38_metal_b200 import Q4RuntimeError

    d = str(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(config, f)
    fixture_index(d, full_map())
    fixture_shard(os.path.join(d, "model.safetensors"))
    with pytest.raises(Q4RuntimeError) as err:
        W.MlxWeightStore(d)
    assert kind_of(err) == kind


def test_projection_spread_over_three_shards_with_odd_header_padding(W, tmp_path, oracle):
    """Weight, scales and biases of one projection may sit in three different shard files (src/native.rs:343-354);
    shards are numbered in name order; offsets are 8 + header length + data offset, whatever the header length."""
    d = str(tmp_path)
    n, k = 24, 256
    w, s, b = oracle.synth_q4(11, 0, n, k)
    norm = oracle.synth_bf16(11, 1, 64)
    f32 = np.arange(6, dtype=np.float32) - 2.5
    W.write_model_dir(d, {
        "model-00002-of-00003.safetensors": {"p.scales": s, "norm.weight": norm},
        "model-00003-of-00003.safetensors": {"p.biases": b, "plain.weight": f32},
        "model-00001-of-00003.safetensors": {"p.weight": w},
    }, header_pad_to=3)
    store = W.MlxWeightStore(d)
    assert store.shard_count() == 3 and store.tensor_count() == 5
    assert store.tensor_names() == sorted(["p.weight", "p.scales", "p.biases", "norm.weight", "plain.weight"])
    assert store.quantized_tensor_groups() == 1  # norm.weight and plain.weight have no companions
    m = store.q4_matrix("p.weight")
    assert (m.input_elements, m.output_rows) == (k, n)
    assert (m.weight.shard_index, m.scales.shard_index, m.biases.shard_index) == (0, 1, 2)
    assert m.weight.byte_offset % 16 == 3 and m.weight.dtype == "U32" and m.weight.shape == (n, k // 8)
    assert store.tensor_data("p.weight") == w.tobytes()
    assert store.tensor_data("p.scales") == s.tobytes()
    assert bytes(store.shard_data(2)[m.biases.byte_offset:m.biases.byte_offset + m.biases.byte_len]) == b.tobytes()
    # tensor_values_f32, src/model.rs:87-112
    np.testing.assert_array_equal(store.tensor_values_f32("norm.weight"), oracle.bf16_to_f32(norm))
    np.testing.assert_array_equal(store.tensor_values_f32("plain.weight"), f32)
    from qwen38_metal_b200 import Q4RuntimeError

    for name, kind in (("p.weight", "UnsupportedRuntimeDtype"), ("absent", "MissingTensor")):
        with pytest.raises(Q4RuntimeError) as err:
            store.tensor_values_f32(name)
        assert kind_of(err) == kind
    for name, kind in (("absent.weight", "MissingTensor"), ("p.scales", "NotQuantizedWeight"), ("norm.weight", "MissingTensor")):
        with pytest.raises(Q4RuntimeError) as err:
            store.q4_matrix(name)
        assert kind_of(err) == kind
    store.close()


def test_json_reader_handles_escapes_and_duplicate_keys(W, tmp_path):
    d = str(tmp_path)
    fixture_config(d)
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        f.write('{"metadata": {"total_size": 1.5e3, "note": "a\\u00e9\\ud83d\\ude00\\n", "flags": [true, false, null]},'
                ' "weight_map": {"t\\u0041": "old.safetensors", "tA": "model.safetensors"}}')
    raw_shard(os.path.join(d, "model.safetensors"), {"tA": {"dtype": "U8", "shape": [2, 2], "data_offsets": [0, 4], "extra": 1}},
              b"\x01\x02\x03\x04")
    store = W.MlxWeightStore(d)
    assert store.tensor_names() == ["tA"] and store.tensor_data("tA") == b"\x01\x02\x03\x04"
    store.close()
