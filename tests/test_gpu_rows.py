"""Short batches (2..16 activation rows) on the integer tensor-core kernel (csrc/q4_gemv_rows.cu): parity against the
scalar oracle at the benchmark's shapes, on ragged row counts, with several projections per call, with fp32
activations, with rows of very different magnitude and through repeated calls (the per-tile counters must be back at
zero after every launch). Bar: relative L2 <= 1e-5, as for a single row."""
import numpy as np
import pytest

from helpers import upload_matrix

pytestmark = pytest.mark.gpu

SEED = 20261


def x_bf16(oracle, tensor, m, k):
    bits = oracle.synth_bf16(SEED, 2000 + tensor, m * k)
    return bits, oracle.bf16_to_f32(bits).reshape(m, k)


@pytest.mark.parametrize("m", [2, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408)])
def test_benchmark_shapes(runtime, oracle, m, n, k):
    trip = oracle.synth_q4(SEED, 1 + (n > k), n, k)
    bits, xf = x_bf16(oracle, m, m, k)
    job = upload_matrix(runtime, *trip)
    out = runtime.q4_affine_matmul_mapped_batch(bits, m, [job])[0]
    assert out.shape == (m, n)
    rows = slice(0, n, 7)  # every seventh output row of every activation row
    ref = oracle.matmul_factored_f32(xf, trip[0][rows], trip[1][rows], trip[2][rows], len(range(n)[rows]), threads=8)
    assert oracle.rel_l2(out[:, rows], ref) <= 1e-5


@pytest.mark.parametrize("m", [2, 5, 8, 12, 16])
def test_ragged_rows_and_several_projections(runtime, oracle, m):
    k = 1536
    shapes = [1000, 53, 16, 1, 300]
    trips = [oracle.synth_q4(SEED, 10 + i, n, k) for i, n in enumerate(shapes)]
    bits, xf = x_bf16(oracle, 20 + m, m, k)
    jobs = [upload_matrix(runtime, *t) for t in trips]
    for _ in range(3):  # counters and scratch carry over between launches
        outs = runtime.q4_affine_matmul_mapped_batch(bits, m, jobs)
        for out, trip, n in zip(outs, trips, shapes):
            assert out.shape == (m, n)
            assert oracle.rel_l2(out, oracle.matmul_factored_f32(xf, *trip, n)) <= 1e-5


@pytest.mark.parametrize("m", [2, 7, 16])
def test_fp32_rows_of_different_magnitude(runtime, oracle, m):
    n, k = 333, 2048
    trip = oracle.synth_q4(SEED, 30, n, k)
    rng = np.random.default_rng(40 + m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x *= (10.0 ** rng.integers(-6, 6, size=(m, 1))).astype(np.float32)  # every row has its own scale
    x[0, : k // 2] = 0.0  # one part of the K range of a row is all zero
    job = upload_matrix(runtime, *trip)
    out = runtime.q4_affine_matmul_mapped_batch(x.reshape(-1), m, [job])[0]
    ref = oracle.matmul_f64(x, *trip, n)
    for r in range(m):
        assert oracle.rel_l2(out[r], ref[r]) <= 1e-5, r


def test_other_shapes_take_the_general_kernels(runtime, oracle):
    """K not a multiple of 512: the fp16 streaming kernel below 16 rows (same bar), the tensor-core GEMM from 16."""
    n, k = 100, 640
    trip = oracle.synth_q4(SEED, 51, n, k)
    job = upload_matrix(runtime, *trip)
    for m, bar in ((4, 1e-5), (16, 2e-3)):
        bits, xf = x_bf16(oracle, 51 + m, m, k)
        out = runtime.q4_affine_matmul_mapped_batch(bits, m, [job])[0]
        assert oracle.rel_l2(out, oracle.matmul_factored_f32(xf, *trip, n)) <= bar


def test_unaligned_tensors_take_the_general_kernel(runtime, oracle):
    n, k, m = 100, 512, 4
    trip = oracle.synth_q4(SEED, 50, n, k)
    bits, xf = x_bf16(oracle, 50, m, k)
    job = upload_matrix(runtime, *trip, offset=2)
    out = runtime.q4_affine_matmul_mapped_batch(bits, m, [job])[0]
    assert oracle.rel_l2(out, oracle.matmul_factored_f32(xf, *trip, n)) <= 1e-5


@pytest.mark.parametrize("m", [2, 8, 16])
def test_residual_form(runtime, oracle, m):
    """out += x W^T (src/metal_runtime.rs matmul_add): the last K part adds to what the caller's buffer holds."""
    k = 2048
    trips = [oracle.synth_q4(SEED, 60 + i, n, k) for i, n in enumerate((333, 48))]
    jobs = [upload_matrix(runtime, *t) for t in trips]
    bits, xf = x_bf16(oracle, 60 + m, m, k)
    res = [np.full((m, t[0].shape[0]), -0.25, dtype=np.float32) for t in trips]
    plain = runtime.q4_affine_matmul_mapped_batch(bits, m, jobs)
    added = runtime.q4_affine_matmul_add_mapped_batch(bits, m, jobs, res)
    for out, add, t in zip(plain, added, trips):
        assert oracle.rel_l2(out, oracle.matmul_factored_f32(xf, *t, t[0].shape[0])) <= 1e-5
        assert np.allclose(add, out - 0.25, rtol=0, atol=1e-6)
