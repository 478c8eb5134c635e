"""Python mirror of the reference's weight store and projection API, over `include/q4b_weights.h`.

`MlxWeightStore`, `Q4AffineMatrix` and `NativeWeights` follow the reference's types of the same names
(src/model.rs:51-134, src/native.rs:208-385, 5383-5471): same method names, argument meaning and error
kinds (`Q4RuntimeError.kind`), so the tests read like the reference's own. The parsing, validation, upload
and every projection run in the C++/CUDA library; nothing is computed here.

`write_safetensors` / `write_model_dir` produce files in the on-disk format (8-byte little-endian header
length, JSON header, data section; `model.safetensors.index.json`; `config.json` with the quantisation
block) for tests and benchmarks -- there is no checkpoint on the machine.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct
from dataclasses import dataclass

import numpy as np

from . import capi
from .runtime import CudaRuntime, _check


@dataclass(frozen=True)
class MlxTensor:
    """src/model.rs:58-65"""

    dtype: str
    shape: tuple
    shard_index: int
    byte_offset: int
    byte_len: int

    @staticmethod
    def from_c(info: capi.TensorInfo) -> "MlxTensor":
        return MlxTensor(info.dtype.decode(), tuple(info.shape[i] for i in range(info.rank)), info.shard_index,
                         info.byte_offset, info.byte_len)

    def to_c(self) -> capi.TensorInfo:
        info = capi.TensorInfo()
        info.dtype = self.dtype.encode()
        info.rank = len(self.shape)
        for i, d in enumerate(self.shape):
            info.shape[i] = d
        info.shard_index, info.byte_offset, info.byte_len = self.shard_index, self.byte_offset, self.byte_len
        return info


class Q4AffineMatrix:
    """src/native.rs:5383-5393. `input_elements` = K, `output_rows` = N (of this rank in a sharded view)."""

    def __init__(self, c: capi.Q4Matrix, name: str):
        self._c = c
        self.weight_name = name
        self.input_elements = c.input_elements
        self.output_rows = c.output_rows
        self.row_begin = c.row_begin
        self.total_rows = c.total_rows

    @property
    def weight(self) -> MlxTensor:
        return MlxTensor.from_c(self._c.weight)

    @property
    def scales(self) -> MlxTensor:
        return MlxTensor.from_c(self._c.scales)

    @property
    def biases(self) -> MlxTensor:
        return MlxTensor.from_c(self._c.biases)

    @staticmethod
    def from_tensors(name: str, weight: MlxTensor, scales: MlxTensor, biases: MlxTensor) -> "Q4AffineMatrix":
        """Q4AffineMatrix::from_tensors, src/native.rs:5419-5471"""
        out = capi.Q4Matrix()
        w, s, b = weight.to_c(), scales.to_c(), biases.to_c()
        _check(capi.load().q4b_q4_matrix_from_tensors(name.encode(), C.byref(w), C.byref(s), C.byref(b), C.byref(out)))
        return Q4AffineMatrix(out, name)


class MlxWeightStore:
    """open_mlx_safetensors_dir + MlxWeightStore, src/model.rs:51-197. Host only: needs no GPU."""

    def __init__(self, path: str, _handle=None):
        self._lib = capi.load()
        self._owned = _handle is None
        if _handle is None:
            _handle = C.c_void_p()
            _check(self._lib.q4b_store_open(os.fsencode(path), C.byref(_handle)))
        self._h = _handle

    def close(self) -> None:
        if self._h and self._owned:
            self._lib.q4b_store_close(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _count(self, fn) -> int:
        out = C.c_uint64()
        _check(fn(self._h, C.byref(out)))
        return out.value

    def tensor_count(self) -> int:
        return self._count(self._lib.q4b_store_tensor_count)

    def shard_count(self) -> int:
        return self._count(self._lib.q4b_store_shard_count)

    def mapped_bytes(self) -> int:
        return self._count(self._lib.q4b_store_mapped_bytes)

    def indexed_tensor_bytes(self) -> int:
        return self._count(self._lib.q4b_store_indexed_tensor_bytes)

    def quantized_tensor_groups(self) -> int:
        return self._count(self._lib.q4b_store_quantized_groups)

    def tensor_names(self) -> list[str]:
        names = []
        for i in range(self.tensor_count()):
            p = C.c_char_p()
            _check(self._lib.q4b_store_tensor_name(self._h, i, C.byref(p)))
            names.append(p.value.decode())
        return names

    def tensor(self, name: str) -> MlxTensor | None:
        info = capi.TensorInfo()
        st = self._lib.q4b_store_tensor(self._h, name.encode(), C.byref(info))
        if st == 24:  # MissingTensor -> Option::None in the reference
            return None
        _check(st)
        return MlxTensor.from_c(info)

    def tensor_data(self, name: str) -> bytes | None:
        data, n = C.c_void_p(), C.c_uint64()
        st = self._lib.q4b_store_tensor_data(self._h, name.encode(), C.byref(data), C.byref(n))
        if st == 24:
            return None
        _check(st)
        return C.string_at(data.value, n.value) if n.value else b""

    def shard_data(self, index: int) -> memoryview:
        data, n = C.c_void_p(), C.c_uint64()
        _check(self._lib.q4b_store_shard_data(self._h, index, C.byref(data), C.byref(n)))
        return memoryview((C.c_uint8 * n.value).from_address(data.value))

    def tensor_values_f32(self, name: str) -> np.ndarray:
        n = C.c_uint64()
        _check(self._lib.q4b_store_tensor_values_f32(self._h, name.encode(), None, 0, C.byref(n)))
        out = np.empty(n.value, dtype=np.float32)
        _check(self._lib.q4b_store_tensor_values_f32(self._h, name.encode(), out.ctypes.data_as(C.c_void_p), n.value, C.byref(n)))
        return out

    def q4_matrix(self, name: str) -> Q4AffineMatrix:
        """Q4AffineMatrix::from_store, src/native.rs:5396-5417"""
        out = capi.Q4Matrix()
        _check(self._lib.q4b_store_q4_matrix(self._h, name.encode(), C.byref(out)))
        return Q4AffineMatrix(out, name)


def _matrices(matrices) -> "C.Array":
    arr = (capi.Q4Matrix * max(len(matrices), 1))()
    for i, m in enumerate(matrices):
        arr[i] = m._c
    return arr


class NativeWeights:
    """NativeWeights, src/native.rs:208-385: the store plus its shards resident in HBM. With `world > 1`
    the view holds this rank's rows of every quantised projection (no reference counterpart)."""

    def __init__(self, path: str, runtime: CudaRuntime, rank: int = 0, world: int = 1):
        self._lib = capi.load()
        self._rt = runtime
        h = C.c_void_p()
        _check(self._lib.q4b_weights_open_sharded(runtime.handle, os.fsencode(path), rank, world, C.byref(h)))
        self._h = h
        sh = C.c_void_p()
        _check(self._lib.q4b_weights_store(self._h, C.byref(sh)))
        self.store = MlxWeightStore(path, _handle=sh)

    @classmethod
    def open(cls, path: str, runtime: CudaRuntime) -> "NativeWeights":
        return cls(path, runtime)

    def close(self) -> None:
        if self._h:
            self._lib.q4b_weights_close(self._h)
            self._h = None
            self.store._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def mapped_shard_count(self) -> int:
        out = C.c_uint64()
        _check(self._lib.q4b_weights_shard_count(self._h, C.byref(out)))
        return out.value

    def device_bytes(self) -> int:
        out = C.c_uint64()
        _check(self._lib.q4b_weights_device_bytes(self._h, C.byref(out)))
        return out.value

    def q4_matrix(self, name: str) -> Q4AffineMatrix:
        out = capi.Q4Matrix()
        _check(self._lib.q4b_weights_q4_matrix(self._h, name.encode(), C.byref(out)))
        return Q4AffineMatrix(out, name)

    def mapped_q4_jobs(self, matrices, input_elements: int) -> list[capi.Job]:
        jobs = (capi.Job * max(len(matrices), 1))()
        _check(self._lib.q4b_weights_jobs(self._h, _matrices(matrices), len(matrices), input_elements, jobs))
        return [jobs[i] for i in range(len(matrices))]

    def q4_affine_matvec(self, matrix: Q4AffineMatrix, x) -> np.ndarray:
        return self.q4_affine_matvec_batch([matrix], x)[0]

    def q4_affine_matvec_batch(self, matrices, x) -> list[np.ndarray]:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        outs = [np.empty(m.output_rows, dtype=np.float32) for m in matrices]
        ptrs = (C.c_void_p * max(len(outs), 1))(*[o.ctypes.data for o in outs])
        _check(self._lib.q4b_weights_matvec_batch(self._h, _matrices(matrices), len(matrices), x.ctypes.data_as(C.c_void_p),
                                                  x.size, ptrs))
        return outs

    def q4_affine_matmul_batch(self, matrices, x, batch_size: int) -> list[np.ndarray]:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        outs = [np.empty((batch_size, m.output_rows), dtype=np.float32) for m in matrices]
        ptrs = (C.c_void_p * max(len(outs), 1))(*[o.ctypes.data for o in outs])
        _check(self._lib.q4b_weights_matmul_batch(self._h, _matrices(matrices), len(matrices), x.ctypes.data_as(C.c_void_p),
                                                  x.size, batch_size, ptrs))
        return outs

    def q4_affine_argmax_batch(self, matrix: Q4AffineMatrix, x, batch_size: int) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        tokens = np.empty(max(batch_size, 1), dtype=np.uint32)
        _check(self._lib.q4b_weights_argmax_batch(self._h, C.byref(matrix._c), x.ctypes.data_as(C.c_void_p), x.size,
                                                  batch_size, tokens.ctypes.data_as(C.c_void_p)))
        return tokens[:batch_size]

    def q4_affine_mlp_batch(self, gate, up, down, x, batch_size: int) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        out = np.empty((max(batch_size, 1), down.output_rows), dtype=np.float32)
        _check(self._lib.q4b_weights_mlp_batch(self._h, C.byref(gate._c), C.byref(up._c), C.byref(down._c),
                                               x.ctypes.data_as(C.c_void_p), x.size, batch_size,
                                               out.ctypes.data_as(C.c_void_p)))
        return out[:batch_size]

    def dequantized_row(self, matrix: Q4AffineMatrix, row: int) -> np.ndarray:
        out = np.empty(matrix.input_elements, dtype=np.float32)
        _check(self._lib.q4b_weights_dequantized_row(self._h, C.byref(matrix._c), row, out.ctypes.data_as(C.c_void_p)))
        return out


# ---- writers (fixtures and benchmark inputs) -------------------------------------------------------

_DTYPES = {np.dtype(np.uint32): "U32", np.dtype(np.float32): "F32", np.dtype(np.uint8): "U8"}


def write_safetensors(path: str, tensors: dict, header_pad_to: int | None = None, dtypes: dict | None = None) -> None:
    """tensors: name -> ndarray (uint16 arrays are written as BF16 unless `dtypes[name]` says otherwise).
    `header_pad_to`: pad the JSON header with spaces so that the data section starts at a file offset congruent
    to this value modulo 16 (real files start their data anywhere; this picks the misalignment)."""
    entries, blobs, pos = {}, [], 0
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        dtype = (dtypes or {}).get(name) or ("BF16" if arr.dtype == np.uint16 else _DTYPES[arr.dtype])
        raw = arr.view(np.uint8).reshape(-1).tobytes()
        entries[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [pos, pos + len(raw)]}
        blobs.append(raw)
        pos += len(raw)
    header = json.dumps(entries, separators=(",", ":")).encode()
    if header_pad_to is not None:
        while (8 + len(header)) % 16 != header_pad_to % 16:
            header += b" "
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)))
        f.write(header)
        for raw in blobs:
            f.write(raw)


def write_model_dir(directory: str, shards: dict, header_pad_to: int | None = None, config: dict | None = None) -> None:
    """shards: shard file name -> {tensor name -> ndarray}. Writes the shards, the weight index and config.json."""
    os.makedirs(directory, exist_ok=True)
    weight_map = {}
    for shard_name, tensors in shards.items():
        write_safetensors(os.path.join(directory, shard_name), tensors, header_pad_to)
        for name in tensors:
            weight_map[name] = shard_name
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(config or {"model_type": "qwen3_5", "quantization_config": {"bits": 4, "group_size": 64, "mode": "affine"}}, f)
