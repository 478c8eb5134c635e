"""The reference's Q4 test fixtures, restated as data.

Each entry reproduces the deterministic input formulas of one test in the reference's
`src/metal_runtime.rs` `mod tests` (line ranges given per case): activations, 4-bit values,
scales and biases are closed-form functions of the flat index. The reference stores no
output vectors; its tests compare the GPU with `cpu_q4_affine_matvec` under an absolute
tolerance (`tol`). `tests/golden/make_golden.py` evaluates the same sums exactly.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from fractions import Fraction

import numpy as np


@dataclass
class Matrix:
    rows: int
    q: tuple[int, int]                 # q[i] = (a*i + b) % 16
    scale: tuple                       # ("const", v) | ("cycle", base, step, period) | ("table", [...])
    bias: tuple


@dataclass
class Case:
    name: str
    ref: str                           # reference lines
    batches: tuple[int, ...]           # batch sizes the test runs
    k: int
    x: tuple[int, int, float]          # x[i] = ((i % p) - c) * step
    matrices: list[Matrix]
    offsets: tuple[int, ...] = (0,)    # byte prefixes exercised (0 = aligned, 1 = the reference's unaligned case)
    tol: float = 1e-3
    kind: str = "matmul"               # matmul | argmax | residual | mlp
    extra: dict = field(default_factory=dict)


S3 = ("cycle", 0.0625, 0.015625, 3)
CASES = [
    Case("matvec_simd", "9332-9367", (1,), 128, (17, 8, 0.125),
         [Matrix(5, (7, 3), ("table", [0.125, -0.0625, 0.25, 0.03125, -0.125, 0.0625]),
                 ("table", [0.03125, -0.015625, 0.0625, 0.125, -0.03125, 0.0]))]),
    Case("batch_two_jobs_one_input", "9685-9763", (1,), 128, (13, 6, 0.125),
         [Matrix(2, (5, 1), ("const", 0.125), ("const", -0.03125)),
          Matrix(4, (3, 7), ("const", 0.0625), ("const", 0.015625))]),
    Case("matmul_each_prompt_row", "9766-9809", (3,), 128, (23, 11, 0.0625),
         [Matrix(3, (7, 5), ("const", 0.125), ("const", -0.03125))]),
    Case("batch_simd_short_batch", "9812-9900", (3,), 512, (37, 18, 0.03125),
         [Matrix(11, (13, 3), S3, ("cycle", -0.015625, 0.0078125, 2))], offsets=(0, 1)),
    Case("batch2_rows2_residual", "9903-10052", (2,), 128, (29, 14, 0.046875),
         [Matrix(5, (11, 3), S3, ("cycle", -0.0234375, 0.0078125, 2))], offsets=(0, 1), kind="residual",
         extra={"initial": (0.125, 0.03125)}),
    Case("unaligned_batch_weight_vectors", "10055-10107", (2, 3), 512, (47, 23, 0.0234375),
         [Matrix(13, (17, 5), ("cycle", 0.046875, 0.0078125, 5), ("cycle", -0.03125, 0.0078125, 4))], offsets=(1,)),
    Case("unaligned_paired_batch_weight_vectors", "10110-10204", (2, 3), 512, (53, 26, 0.01953125),
         [Matrix(11, (7, 3), S3, ("cycle", -0.0234375, 0.0078125, 2)),
          Matrix(7, (13, 9), ("cycle", 0.0390625, 0.0078125, 4), ("cycle", -0.015625, 0.00390625, 3))],
         offsets=(1,)),
    Case("batch_simd_pair_short_batch", "10207-10325", (3,), 512, (41, 20, 0.0234375),
         [Matrix(11, (7, 1), S3, ("cycle", -0.03125, 0.0078125, 2)),
          Matrix(7, (11, 5), ("cycle", 0.046875, 0.01171875, 4), ("cycle", -0.0234375, 0.00390625, 3))]),
    Case("short_pair_batch", "10328-10450", (2, 3), 128, (31, 15, 0.046875),
         [Matrix(37, (7, 1), S3, ("cycle", -0.03125, 0.0078125, 2)),
          Matrix(29, (11, 5), ("cycle", 0.046875, 0.01171875, 4), ("cycle", -0.0234375, 0.00390625, 3))]),
    Case("argmax_batch", "10453-10500", (3,), 128, (29, 14, 0.046875),
         [Matrix(37, (13, 7), S3, ("cycle", -0.0234375, 0.0078125, 2))], kind="argmax", tol=0.0),
    Case("short_matmul_unaligned_batch", "10503-10558", (5,), 128, (29, 14, 0.046875),
         [Matrix(5, (11, 3), ("const", 0.09375), ("const", -0.0234375))], offsets=(1,)),
    Case("mapped_matmul_unaligned_prompt_rows", "10561-10618", (256,), 128, (31, 15, 0.046875),
         [Matrix(3, (9, 2), ("const", 0.09375), ("const", -0.0234375))], offsets=(1,), tol=0.08),
    Case("simdgroup_matmul_batch", "10621-10673", (64,), 128, (37, 18, 0.03125),
         [Matrix(11, (5, 9), S3, ("cycle", -0.015625, 0.0078125, 2))], tol=0.08),
    Case("wide_simdgroup_matmul_batch", "10676-10723", (3072,), 128, (41, 20, 0.0234375),
         [Matrix(19, (13, 2), ("cycle", 0.046875, 0.01171875, 4), ("cycle", -0.01171875, 0.00390625, 3))], tol=0.08),
    Case("fused_mlp_batch", "10726-10910", (256, 1), 64, (29, 14, 0.03125),
         [Matrix(64, (5, 1), ("const", 0.0625), ("const", -0.015625)),      # gate
          Matrix(64, (11, 3), ("const", 0.03125), ("const", 0.0078125)),    # up
          Matrix(64, (13, 7), ("const", 0.125), ("const", -0.03125))],      # down (input width 64)
         kind="mlp", tol=0.15, extra={"decode_tol": 1e-3}),
]


def _param_values(spec, count: int) -> list[float]:
    if spec[0] == "const":
        return [spec[1]] * count
    if spec[0] == "cycle":
        _, base, step, period = spec
        return [float(np.float32(base) + np.float32(i % period) * np.float32(step)) for i in range(count)]
    if spec[0] == "table":
        return [spec[1][i % len(spec[1])] for i in range(count)]
    raise ValueError(spec)


def f32_to_bf16(values) -> np.ndarray:
    """f32_to_bf16 of the reference's tests (src/metal_runtime.rs:12128-12132)."""
    bits = np.asarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFFFFFF) >> 16).astype(np.uint16)


def bf16_to_f32(bits) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def pack_q4(q: np.ndarray) -> np.ndarray:
    """pack_q4 of the reference's tests (src/metal_runtime.rs:11962-11975)."""
    q = np.asarray(q, dtype=np.uint32).reshape(-1, 8)
    out = np.zeros(q.shape[0], dtype=np.uint32)
    for i in range(8):
        out |= q[:, i] << np.uint32(4 * i)
    return out


def case_input(case: Case, batch: int) -> np.ndarray:
    p, c, step = case.x
    i = np.arange(batch * case.k)
    return (((i % p).astype(np.float32) - np.float32(c)) * np.float32(step)).reshape(batch, case.k)


def matrix_tensors(m: Matrix, k: int):
    """(q uint8 [rows][k], packed u32 [rows][k/8], scales u16 [rows][k/64], biases u16 [rows][k/64])."""
    i = np.arange(m.rows * k)
    q = ((i * m.q[0] + m.q[1]) % 16).astype(np.uint8).reshape(m.rows, k)
    groups = k // 64
    scales = f32_to_bf16(_param_values(m.scale, m.rows * groups)).reshape(m.rows, groups)
    biases = f32_to_bf16(_param_values(m.bias, m.rows * groups)).reshape(m.rows, groups)
    return q, pack_q4(q).reshape(m.rows, k // 8), scales, biases


def prefixed(arr: np.ndarray, offset: int) -> np.ndarray:
    """prefixed_u32_bytes / prefixed_u16_bytes (src/metal_runtime.rs:11944-11960): `offset` zero bytes, then data."""
    raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
    return np.concatenate([np.zeros(offset, dtype=np.uint8), raw])


def exact_projection(case: Case, batch: int, q: np.ndarray, scales: np.ndarray, biases: np.ndarray) -> np.ndarray:
    """sum_k x*(q*scale+bias) evaluated exactly, rounded once to float64. Returns [batch][rows].

    x = integer * step, q integer, scale/bias dyadic rationals: the per-group sums are integer dot
    products and only the last combination needs rationals.
    """
    p, c, step = case.x
    k = case.k
    rows, groups = q.shape[0], k // 64
    i = np.arange(batch * k)
    xint = ((i % p) - c).astype(np.int64).reshape(batch, groups, 64)
    qg = q.astype(np.int64).reshape(rows, groups, 64)
    dots = np.einsum("bgk,rgk->brg", xint, qg)          # exact in int64
    sums = xint.sum(axis=2)                              # [batch][groups]
    sf = [[Fraction(float(v)) for v in row] for row in bf16_to_f32(scales).reshape(rows, groups)]
    bf = [[Fraction(float(v)) for v in row] for row in bf16_to_f32(biases).reshape(rows, groups)]
    stepf = Fraction(float(np.float32(step)))
    out = np.empty((batch, rows), dtype=np.float64)
    cache: dict = {}
    for b in range(batch):
        key = (b * k) % p                                # rows of x repeat with the index pattern
        if key not in cache:
            vals = []
            for r in range(rows):
                total = Fraction(0)
                for g in range(groups):
                    total += sf[r][g] * int(dots[b, r, g]) + bf[r][g] * int(sums[b, g])
                vals.append(float(total * stepf))
            cache[key] = vals
        out[b] = cache[key]
    return out
