"""NativeWeights on the GPU: safetensors files on disk -> shards in HBM -> projections, against the CPU oracle.

Mirrors how the reference's model code uses the path (src/native.rs:216-323): open a directory, ask for matrices by
tensor name, run grouped projections. Files are written with a header length that leaves every tensor two bytes off
a 4-byte boundary, which is the case the byte-addressed kernels exist for.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HIDDEN, INTER, VOCAB = 512, 320, 1000
ROWS = {"q_proj": 96, "k_proj": 32, "v_proj": 32, "tiny": 2}


@pytest.fixture(scope="module")
def model(tmp_path_factory, oracle):
    from qwen38_metal_b200 import weights as W

    d = str(tmp_path_factory.mktemp("model"))
    tensors, shards = {}, {"model-00001-of-00002.safetensors": {}, "model-00002-of-00002.safetensors": {}}
    specs = [(f"layers.0.attn.{n}", rows, HIDDEN) for n, rows in ROWS.items()]
    specs += [("layers.0.mlp.gate_proj", INTER, HIDDEN), ("layers.0.mlp.up_proj", INTER, HIDDEN),
              ("layers.0.mlp.down_proj", HIDDEN, INTER), ("lm_head", VOCAB, HIDDEN)]
    for i, (name, n, k) in enumerate(specs):
        w, s, b = oracle.synth_q4(5, i, n, k)
        tensors[name] = (w, s, b, n, k)
        first = shards["model-00001-of-00002.safetensors"]
        second = shards["model-00002-of-00002.safetensors"]
        # scales of every other projection live in the other shard file
        first[name + ".weight"] = w
        (second if i % 2 else first)[name + ".scales"] = s
        first[name + ".biases"] = b
    shards["model-00002-of-00002.safetensors"]["norm.weight"] = oracle.synth_bf16(5, 99, HIDDEN)
    W.write_model_dir(d, shards, header_pad_to=2)
    return d, tensors


def activation(oracle, seed, rows=1):
    return oracle.bf16_to_f32(oracle.synth_bf16(seed, 1000, rows * HIDDEN)).reshape(rows, HIDDEN)


def test_open_and_grouped_matvec(runtime, oracle, model):
    from qwen38_metal_b200 import Q4RuntimeError
    from qwen38_metal_b200.weights import NativeWeights

    d, tensors = model
    nw = NativeWeights.open(d, runtime)
    assert nw.mapped_shard_count() == 2 and nw.device_bytes() == nw.store.mapped_bytes()
    names = [f"layers.0.attn.{n}" for n in ROWS]
    mats = [nw.q4_matrix(n + ".weight") for n in names]
    assert mats[0].weight.byte_offset % 4 == 2  # the files really are misaligned
    jobs = nw.mapped_q4_jobs(mats, HIDDEN)
    assert [j.aligned for j in jobs] == [0] * len(jobs)
    x = activation(oracle, 7)[0]
    outs = nw.q4_affine_matvec_batch(mats, x)
    for name, y in zip(names, outs):
        w, s, b, n, k = tensors[name]
        assert oracle.rel_l2(y, oracle.matmul_f64(x, w, s, b, n)[0]) <= 1e-5
    np.testing.assert_array_equal(nw.q4_affine_matvec(mats[1], x), outs[1])
    with pytest.raises(Q4RuntimeError) as err:
        nw.q4_affine_matvec_batch(mats, x[:448])
    assert err.value.kind == "InputDimension"
    with pytest.raises(Q4RuntimeError) as err:
        nw.q4_affine_matvec_batch([], x)
    assert err.value.kind == "InvalidConfig"
    with pytest.raises(Q4RuntimeError) as err:
        nw.q4_matrix("norm.weight")
    assert err.value.kind == "MissingTensor"
    nw.close()


def test_prefill_argmax_mlp_and_row_lookup(runtime, oracle, model):
    from qwen38_metal_b200 import Q4RuntimeError
    from qwen38_metal_b200.weights import NativeWeights

    d, tensors = model
    nw = NativeWeights.open(d, runtime)
    m = 5
    x = activation(oracle, 8, m)
    gate, up, down, head = (nw.q4_matrix(f"{n}.weight") for n in
                            ("layers.0.mlp.gate_proj", "layers.0.mlp.up_proj", "layers.0.mlp.down_proj", "lm_head"))
    outs = nw.q4_affine_matmul_batch([gate, up], x, m)
    for name, y in zip(("layers.0.mlp.gate_proj", "layers.0.mlp.up_proj"), outs):
        w, s, b, n, k = tensors[name]
        assert y.shape == (m, n) and oracle.rel_l2(y, oracle.matmul_f64(x, w, s, b, n)) <= 1e-5
    w, s, b, n, k = tensors["lm_head"]
    logits = oracle.matmul_factored_f32(x, w, s, b, n)
    tokens = nw.q4_affine_argmax_batch(head, x, m)
    assert tokens.dtype == np.uint32
    for row, tok in enumerate(tokens):  # the winner's logit is the row maximum (summation order may move near-ties)
        assert logits[row, tok] >= logits[row].max() - 1e-4 * abs(logits[row].max())
    g, u, dn = (tensors[f"layers.0.mlp.{p}_proj"][:3] for p in ("gate", "up", "down"))
    y = nw.q4_affine_mlp_batch(gate, up, down, x, m)
    assert oracle.rel_l2(y, oracle.mlp(x, g, u, dn, INTER, HIDDEN)) <= 4e-3  # the intermediate is held as bf16
    for row in (0, 17, VOCAB - 1):
        np.testing.assert_array_equal(nw.dequantized_row(head, row), oracle.dequantize_row(w, s, b, HIDDEN, row))
    with pytest.raises(Q4RuntimeError) as err:
        nw.dequantized_row(head, VOCAB)
    assert err.value.kind == "TokenOutOfRange"
    for bad_batch in (0, 3):  # 5 rows of 512 do not split into 3 equal rows
        with pytest.raises(Q4RuntimeError) as err:
            nw.q4_affine_matmul_batch([gate], x, bad_batch)
        assert err.value.kind == "InvalidConfig"
    job = nw.mapped_q4_jobs([head], HIDDEN)[0]
    nw.close()
    # the shards are gone with the weights: their ids no longer resolve
    from qwen38_metal_b200.runtime import _check

    out = np.zeros(VOCAB, dtype=np.float32)
    import ctypes as C

    with pytest.raises(Q4RuntimeError) as err:
        _check(runtime._lib.q4b_dequantize_row(runtime.handle, C.byref(job), HIDDEN, 0, out.ctypes.data_as(C.c_void_p)))
    assert err.value.kind == "MissingMappedShard"


@pytest.mark.parametrize("world", [2, 3])
def test_row_sharded_views_reassemble_bit_exactly(runtime, oracle, model, world):
    """Each rank uploads only its rows; the pieces put side by side equal the unsharded outputs bit for bit
    (a row's reduction order does not depend on which other rows share the launch)."""
    from qwen38_metal_b200 import Q4RuntimeError
    from qwen38_metal_b200.weights import NativeWeights

    d, tensors = model
    whole = NativeWeights.open(d, runtime)
    names = ["layers.0.attn.q_proj", "layers.0.attn.k_proj", "layers.0.mlp.gate_proj", "lm_head"]
    x = activation(oracle, 9)[0]
    expect = whole.q4_affine_matvec_batch([whole.q4_matrix(n + ".weight") for n in names], x)
    total_bytes = 0
    pieces = {n: [] for n in names}
    for rank in range(world):
        view = NativeWeights(d, runtime, rank=rank, world=world)
        total_bytes += view.device_bytes()
        mats = [view.q4_matrix(n + ".weight") for n in names]
        for n, m in zip(names, mats):
            rows = tensors[n][3]
            assert (m.row_begin, m.output_rows, m.total_rows) == (rows * rank // world, rows * (rank + 1) // world - rows * rank // world, rows)
            # the slice keeps the file's address modulo 16
            src = whole.q4_matrix(n + ".weight")
            assert m.weight.byte_offset % 16 == (src.weight.byte_offset + m.row_begin * (HIDDEN // 2)) % 16
        for n, y in zip(names, view.q4_affine_matvec_batch(mats, x)):
            pieces[n].append(y)
        tiny = view.q4_matrix("layers.0.attn.tiny.weight")  # two rows over three ranks: someone gets none
        if tiny.output_rows == 0:
            with pytest.raises(Q4RuntimeError) as err:
                view.mapped_q4_jobs([tiny], HIDDEN)
            assert err.value.kind == "EmptyDimension"
        else:
            view.q4_affine_matvec(tiny, x)
        view.close()
    for n, y in zip(names, expect):
        np.testing.assert_array_equal(np.concatenate(pieces[n]), y)
    # every projection byte is uploaded exactly once over the ranks; the replicated norm vector once per rank
    quant = sum(w.nbytes + s.nbytes + b.nbytes for (w, s, b, _, _) in tensors.values())
    assert total_bytes == quant + world * HIDDEN * 2
    whole.close()
