"""Format-level properties of the oracle: packing is bit exact, the quantiser follows the recipe,
the three arithmetic forms agree, and the threaded driver equals the scalar one."""
import numpy as np

import ref_cases as rc


def test_pack_unpack_round_trip_bit_exact(oracle):
    rng = np.random.default_rng(7)
    q = rng.integers(0, 16, size=64 * 40, dtype=np.uint8)
    words = oracle.pack(q)
    assert np.array_equal(oracle.unpack(words), q)
    assert np.array_equal(words, rc.pack_q4(q))  # numpy restatement of pack_q4
    # nibble i of a word is value i (low nibble first), little-endian bytes
    one = oracle.pack(np.arange(8, dtype=np.uint8))
    assert one[0] == 0x76543210
    assert one.view(np.uint8).tolist() == [0x10, 0x32, 0x54, 0x76]


def test_bf16_round_to_nearest_even(oracle):
    vals = np.array([1.0, 1.00390625, 1.01171875, -0.0625, 3.140625, 1e-30, 65504.0], dtype=np.float32)
    ours = oracle.f32_to_bf16(vals)
    assert np.array_equal(ours, rc.f32_to_bf16(vals))
    for v, b in zip(vals, ours):
        assert oracle.lib().q4o_f32_to_bf16(float(v)) == int(b)
    # 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7: even mantissa wins
    assert oracle.f32_to_bf16(np.array([1.00390625], dtype=np.float32))[0] == 0x3F80
    assert oracle.f32_to_bf16(np.array([1.01171875], dtype=np.float32))[0] == 0x3F82


def test_quantiser_follows_recipe(oracle):
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((6, 256)) * 0.02).astype(np.float32)
    w[3, 64:128] = 0.5  # constant group: scale 0, q 0
    words, scales, biases = oracle.quantize(w)
    q = oracle.unpack(words).reshape(6, 256)
    g = w.reshape(6, 4, 64)
    lo, hi = g.min(axis=2), g.max(axis=2)
    scale = ((hi - lo) / np.float32(15.0)).astype(np.float32)
    assert np.array_equal(scales, rc.f32_to_bf16(scale))
    assert np.array_equal(biases, rc.f32_to_bf16(lo))
    with np.errstate(divide="ignore", invalid="ignore"):
        expect = np.where(scale[..., None] != 0, np.rint((g - lo[..., None]) / scale[..., None]), 0)
    assert np.array_equal(q.reshape(6, 4, 64), np.clip(expect, 0, 15).astype(np.uint8))
    assert np.all(q[3, 64:128] == 0) and scales[3, 1] == 0
    # every group uses the whole range
    assert q.reshape(6, 4, 64).max(axis=2)[scale != 0].min() == 15


def test_forms_agree_on_random_inputs(oracle):
    words, scales, biases = oracle.synth_q4(1234, 5, 48, 1024)
    x = oracle.bf16_to_f32(oracle.synth_bf16(1234, 99, 3 * 1024)).reshape(3, 1024)
    truth = oracle.matmul_f64(x, words, scales, biases, 48)
    factored = oracle.matmul_factored_f32(x, words, scales, biases, 48)
    dequant = oracle.matmul_dequant_f32(x, words, scales, biases, 48)
    tiles = oracle.matmul_bf16_tiles(x, words, scales, biases, 48)
    assert oracle.rel_l2(factored, truth) < 1e-6
    assert oracle.rel_l2(dequant, truth) < 1e-6
    # rounding the dequantised weight to bf16 costs about 2^-9/sqrt(3)
    assert 1e-4 < oracle.rel_l2(tiles, truth) < 2e-3
    threaded = oracle.matmul_factored_f32(x, words, scales, biases, 48, threads=4)
    assert np.array_equal(threaded, factored)


def test_numpy_restatement_of_the_format(oracle):
    words, scales, biases = oracle.synth_q4(77, 1, 10, 192)  # three groups per row: odd group count
    x = oracle.bf16_to_f32(oracle.synth_bf16(77, 2, 192))
    q = ((words[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).reshape(10, 192).astype(np.float64)
    w = q * oracle.bf16_to_f32(scales).astype(np.float64).repeat(64, axis=1) \
        + oracle.bf16_to_f32(biases).astype(np.float64).repeat(64, axis=1)
    assert np.allclose(oracle.matmul_f64(x, words, scales, biases, 10)[0], w @ x.astype(np.float64), rtol=1e-12, atol=1e-12)
    assert np.allclose(oracle.dequantize_row(words, scales, biases, 192, 4), w[4].astype(np.float32))


def test_byte_offsets_do_not_change_results(oracle):
    words, scales, biases = oracle.synth_q4(5, 3, 7, 128)
    x = oracle.bf16_to_f32(oracle.synth_bf16(5, 4, 128))
    base = oracle.matmul_factored_f32(x, words, scales, biases, 7)
    for off in (1, 2, 3, 4, 8):
        got = oracle.matmul_factored_f32(x, rc.prefixed(words, off)[off:], rc.prefixed(scales, off)[off:],
                                         rc.prefixed(biases, off)[off:], 7)
        assert np.array_equal(got, base)


def test_synthetic_generator_is_deterministic_and_row_addressable(oracle):
    a = oracle.synth_q4(42, 9, 16, 128)
    b = oracle.synth_q4(42, 9, 16, 128)
    assert all(np.array_equal(u, v) for u, v in zip(a, b))
    tail = oracle.synth_q4(42, 9, 6, 128, row0=10)  # rows 10..15 generated on their own
    assert all(np.array_equal(u[10:], v) for u, v in zip(a, tail))
    other = oracle.synth_q4(43, 9, 16, 128)
    assert not np.array_equal(a[0], other[0])
    vals = np.array([oracle.lib().q4o_synth_normal(42, 1, i) for i in range(20000)])
    assert abs(vals.mean()) < 0.03 and abs(vals.std() - 1.0) < 0.03
