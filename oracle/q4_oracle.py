"""ctypes front end of the CPU oracle (oracle/q4_oracle.c) -- TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
The product package never does: it has no CPU path at all.

Arrays are numpy; weights/scales/biases are passed as uint8 byte views so any byte
alignment can be exercised (the reference's `_unaligned` kernels read byte-wise,
shaders/qwen38.metal:105-115).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libq4oracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "q4_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s"])
    return _LIB_PATH


def _load():
    if not os.path.exists(_LIB_PATH):
        build()
    lib = C.CDLL(_LIB_PATH)
    sz, p, f32p = C.c_size_t, C.c_void_p, C.c_void_p
    mm = [f32p, sz, sz, p, p, p, sz, p]
    for name in ("q4o_matmul_dequant_f32", "q4o_matmul_factored_f32", "q4o_matmul_f64", "q4o_matmul_bf16_tiles"):
        getattr(lib, name).argtypes = mm
        getattr(lib, name).restype = None
    for name in ("q4o_matmul_factored_f32_mt", "q4o_matmul_bf16_tiles_mt"):
        getattr(lib, name).argtypes = mm + [C.c_int]
        getattr(lib, name).restype = None
    lib.q4o_pack.argtypes = [p, sz, p]
    lib.q4o_unpack.argtypes = [p, sz, p]
    lib.q4o_quantize.argtypes = [p, sz, sz, p, p, p]
    lib.q4o_argmax_rows.argtypes = [p, sz, sz, p]
    lib.q4o_swiglu.argtypes = [p, p, sz, p]
    lib.q4o_mlp.argtypes = [p, sz, sz, p, p, p, p, p, p, sz, p, p, p, sz, C.c_int, p]
    lib.q4o_dequantize_row.argtypes = [p, p, p, sz, sz, p]
    lib.q4o_f32_to_bf16.argtypes = [C.c_float]
    lib.q4o_f32_to_bf16.restype = C.c_uint16
    lib.q4o_bf16_to_f32.argtypes = [C.c_uint16]
    lib.q4o_bf16_to_f32.restype = C.c_float
    lib.q4o_splitmix64.argtypes = [C.c_uint64]
    lib.q4o_splitmix64.restype = C.c_uint64
    lib.q4o_synth_normal.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64]
    lib.q4o_synth_normal.restype = C.c_float
    lib.q4o_synth_q4_rows.argtypes = [C.c_uint64, C.c_uint64, C.c_float, sz, sz, sz, p, p, p]
    lib.q4o_synth_bf16.argtypes = [C.c_uint64, C.c_uint64, sz, p]
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _bytes(a) -> np.ndarray:
    """uint8 view of a tensor's bytes, keeping the caller's (possibly odd) alignment."""
    a = np.asarray(a)
    if a.dtype != np.uint8:
        a = np.ascontiguousarray(a).view(np.uint8)
    return a.reshape(-1)


def f32_to_bf16(x) -> np.ndarray:
    """RNE without a NaN case (src/metal_runtime.rs:12128-12132), vectorised."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFFFFFF
    return (rounded >> 16).astype(np.uint16)


def bf16_to_f32(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def pack(q) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8).reshape(-1)
    out = np.empty(q.size // 8, dtype=np.uint32)
    lib().q4o_pack(_ptr(q), q.size, _ptr(out))
    return out


def unpack(words) -> np.ndarray:
    words = np.ascontiguousarray(words, dtype=np.uint32).reshape(-1)
    out = np.empty(words.size * 8, dtype=np.uint8)
    lib().q4o_unpack(_ptr(words), words.size, _ptr(out))
    return out


def quantize(w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    words = np.empty((rows, cols // 8), dtype=np.uint32)
    scales = np.empty((rows, cols // 64), dtype=np.uint16)
    biases = np.empty((rows, cols // 64), dtype=np.uint16)
    lib().q4o_quantize(_ptr(w), rows, cols, _ptr(words), _ptr(scales), _ptr(biases))
    return words, scales, biases


def _matmul(name, x, weights, scales, biases, n, out_dtype=np.float32, threads=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim == 1:
        x = x[None, :]
    m, k = x.shape
    wb, sb, bb = _bytes(weights), _bytes(scales), _bytes(biases)
    assert wb.size >= n * k // 2 and sb.size >= n * (k // 64) * 2 and bb.size >= n * (k // 64) * 2
    y = np.empty((m, n), dtype=out_dtype)
    args = [_ptr(x), m, k, _ptr(wb), _ptr(sb), _ptr(bb), n, _ptr(y)]
    if threads is not None:
        args.append(int(threads))
    getattr(lib(), name)(*args)
    return y


def matmul_dequant_f32(x, w, s, b, n):
    return _matmul("q4o_matmul_dequant_f32", x, w, s, b, n)


def matmul_factored_f32(x, w, s, b, n, threads=None):
    if threads is None:
        return _matmul("q4o_matmul_factored_f32", x, w, s, b, n)
    return _matmul("q4o_matmul_factored_f32_mt", x, w, s, b, n, threads=threads)


def matmul_f64(x, w, s, b, n):
    return _matmul("q4o_matmul_f64", x, w, s, b, n, out_dtype=np.float64)


def matmul_bf16_tiles(x, w, s, b, n, threads=None):
    if threads is None:
        return _matmul("q4o_matmul_bf16_tiles", x, w, s, b, n)
    return _matmul("q4o_matmul_bf16_tiles_mt", x, w, s, b, n, threads=threads)


def argmax_rows(logits) -> np.ndarray:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    m, n = logits.shape
    out = np.empty(m, dtype=np.uint32)
    lib().q4o_argmax_rows(_ptr(logits), m, n, _ptr(out))
    return out


def swiglu(gate, up) -> np.ndarray:
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(gate)
    lib().q4o_swiglu(_ptr(gate), _ptr(up), gate.size, _ptr(out))
    return out


def mlp(x, gate, up, down, inter, n, form=0) -> np.ndarray:
    """gate/up/down are (weights, scales, biases) triples."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim == 1:
        x = x[None, :]
    m, k = x.shape
    y = np.empty((m, n), dtype=np.float32)
    g, u, d = ([_bytes(t) for t in trip] for trip in (gate, up, down))
    lib().q4o_mlp(_ptr(x), m, k, _ptr(g[0]), _ptr(g[1]), _ptr(g[2]), _ptr(u[0]), _ptr(u[1]), _ptr(u[2]),
                  inter, _ptr(d[0]), _ptr(d[1]), _ptr(d[2]), n, form, _ptr(y))
    return y


def dequantize_row(w, s, b, k, row) -> np.ndarray:
    out = np.empty(k, dtype=np.float32)
    wb, sb, bb = _bytes(w), _bytes(s), _bytes(b)
    lib().q4o_dequantize_row(_ptr(wb), _ptr(sb), _ptr(bb), k, row, _ptr(out))
    return out


def synth_q4(seed, tensor, n, k, sigma=0.02, row0=0):
    words = np.empty((n, k // 8), dtype=np.uint32)
    scales = np.empty((n, k // 64), dtype=np.uint16)
    biases = np.empty((n, k // 64), dtype=np.uint16)
    lib().q4o_synth_q4_rows(seed, tensor, sigma, row0, n, k, _ptr(words), _ptr(scales), _ptr(biases))
    return words, scales, biases


def synth_bf16(seed, tensor, count) -> np.ndarray:
    out = np.empty(count, dtype=np.uint16)
    lib().q4o_synth_bf16(seed, tensor, count, _ptr(out))
    return out


def rel_l2(actual, expected) -> float:
    a = np.asarray(actual, dtype=np.float64).reshape(-1)
    e = np.asarray(expected, dtype=np.float64).reshape(-1)
    denom = float(np.linalg.norm(e))
    return float(np.linalg.norm(a - e)) / (denom if denom > 0 else 1.0)
