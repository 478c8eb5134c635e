"""ctypes prototypes of include/q4b200.h and include/q4b_weights.h. The library is required: there is no fallback."""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

Q4B_F32, Q4B_BF16 = 0, 1
FLAG_ACCUMULATE, FLAG_STREAM, FLAG_TENSOR = 1, 2, 4

STATUS_NAMES = {
    0: "Ok", 1: "NoDevice", 2: "EmptyBuffer", 3: "ActivationPoolPoisoned", 4: "EmptyDimension",
    5: "InputNotGrouped", 6: "WrongLength", 7: "MissingMappedShard", 8: "InvalidBufferOffset",
    9: "MappedTensorOutOfRange", 10: "DimensionOverflow", 11: "CommandFailed", 12: "CudaError",
    13: "InvalidArgument", 14: "Unsupported", 15: "Read", 16: "Json", 17: "MissingQuantization",
    18: "UnsupportedQuantization", 19: "UnsafeShardPath", 20: "InvalidHeaderLength", 21: "MissingIndexedTensor",
    22: "InvalidTensorOffsets", 23: "InvalidTensorMetadata", 24: "MissingTensor", 25: "InvalidRuntimeTensor",
    26: "UnsupportedRuntimeDtype", 27: "IncompleteAffineGroup", 28: "NotQuantizedWeight",
    29: "InvalidQuantizedWeight", 30: "InvalidAffineTensor", 31: "TensorByteLength", 32: "InputDimension",
    33: "InvalidConfig", 34: "TokenOutOfRange",
}


class Job(C.Structure):
    """q4b_job: MappedQ4AffineJob of the reference (src/metal_runtime.rs:155-192)."""

    _fields_ = [
        ("weight_shard", C.c_uint32), ("scale_shard", C.c_uint32), ("bias_shard", C.c_uint32),
        ("aligned", C.c_int32),
        ("weight_offset", C.c_uint64), ("scale_offset", C.c_uint64), ("bias_offset", C.c_uint64),
        ("output_rows", C.c_uint64),
    ]


class TensorInfo(C.Structure):
    """q4b_tensor_info: MlxTensor of the reference (src/model.rs:58-65)."""

    _fields_ = [
        ("dtype", C.c_char * 16), ("rank", C.c_uint32), ("shard_index", C.c_uint32), ("shape", C.c_uint64 * 8),
        ("byte_offset", C.c_uint64), ("byte_len", C.c_uint64),
    ]


class Q4Matrix(C.Structure):
    """q4b_q4_matrix: Q4AffineMatrix of the reference (src/native.rs:5383-5393)."""

    _fields_ = [
        ("weight", TensorInfo), ("scales", TensorInfo), ("biases", TensorInfo),
        ("input_elements", C.c_uint64), ("output_rows", C.c_uint64), ("row_begin", C.c_uint64), ("total_rows", C.c_uint64),
    ]


class Stage(C.Structure):
    """q4b_stage: one stage of the persistent decode chain."""

    _fields_ = [
        ("x_kind", C.c_uint32), ("eps", C.c_float), ("k", C.c_uint64),
        ("src0", C.c_void_p), ("src1", C.c_void_p), ("x_bf16_out", C.c_void_p),
        ("jobs", C.POINTER(Job)), ("n_jobs", C.c_uint32), ("outputs", C.POINTER(C.c_void_p)),
        ("peer_outputs", C.POINTER(C.c_void_p)),
        ("k_total", C.c_uint64), ("k_begin", C.c_uint64), ("src_parts", C.c_uint32), ("reserved", C.c_uint32),
        ("src_part_stride", C.c_uint64), ("sum_out", C.c_void_p),
    ]


class Peers(C.Structure):
    """q4b_peers: the ranks of a row-sharded chain."""

    _fields_ = [("world", C.c_uint32), ("rank", C.c_uint32), ("flags", C.c_void_p * 8), ("cand", C.c_void_p * 8)]


X_BF16, X_SWIGLU, X_RMS = 0, 1, 2

_lib = None


def library_path() -> str:
    return _build.LIB_PATH


def load() -> C.CDLL:
    """Load lib/libq4b200.so, or raise: the package has no other compute path."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m qwen38_metal_b200.build` "
            "(the package has no CPU or PyTorch fallback)")
    lib = C.CDLL(path)
    vp, u32, u64, i32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int
    P = C.POINTER
    sig = {
        "q4b_runtime_create": [i32, P(vp)],
        "q4b_device_info": [vp, P(i32), P(u64), C.c_char_p, u32],
        "q4b_shard_upload": [vp, vp, u64, P(u32)],
        "q4b_shard_alloc": [vp, u64, P(u32)],
        "q4b_shard_write": [vp, u32, u64, vp, u64],
        "q4b_shard_read": [vp, u32, u64, vp, u64],
        "q4b_shard_count": [vp, P(u32)],
        "q4b_shard_info": [vp, u32, P(vp), P(u64)],
        "q4b_offset_is_aligned": [vp, u32, u64, u64, P(i32)],
        "q4b_matvec_batch": [vp, vp, i32, u64, P(Job), u32, P(vp)],
        "q4b_matmul_batch": [vp, vp, i32, u64, u64, P(Job), u32, P(vp)],
        "q4b_matmul_add_batch": [vp, vp, i32, u64, u64, P(Job), u32, P(vp)],
        "q4b_argmax_batch": [vp, vp, i32, u64, u64, P(Job), vp],
        "q4b_mlp_batch": [vp, vp, i32, u64, u64, P(Job), P(Job), P(Job), vp],
        "q4b_dequantize_row": [vp, P(Job), u64, u64, vp],
        "q4b_matmul_batch_device": [vp, vp, i32, u64, u64, P(Job), u32, P(vp), u32, vp],
        "q4b_mlp_batch_device": [vp, vp, i32, u64, u64, P(Job), P(Job), P(Job), vp, vp],
        "q4b_argmax_batch_device": [vp, vp, i32, u64, u64, P(Job), u32, vp, vp, vp],
        "q4b_swiglu_device": [vp, vp, vp, u64, vp, vp, vp],
        "q4b_rms_unit_bf16_device": [vp, vp, u32, u32, C.c_float, vp, vp],
        "q4b_synth_q4_device": [vp, u64, u64, C.c_float, u64, u64, u64, P(Job)],
        "q4b_synth_bf16_device": [vp, u64, u64, u64, vp, vp],
        "q4b_describe_dispatch": [vp, i32, u64, u64, P(Job), u32, C.c_char_p, u32],
        "q4b_launch_count": [vp, P(u64)],
        "q4b_profile_begin": [vp],
        "q4b_trace_enable": [vp, i32],
        "q4b_trace_read": [vp, vp, u32, P(u32)],
        "q4b_profile_end": [vp, P(u64), P(C.c_double), P(u64), P(u64)],
        "q4b_device_status": [vp],
        "q4b_chain_create": [vp, P(Stage), u32, vp, u32, u32, vp, vp, P(Peers), P(vp)],
        "q4b_arena_create": [vp, u64, P(vp), C.c_char_p],
        "q4b_arena_open": [vp, C.c_char_p, P(vp)],
        "q4b_chain_run_device": [vp, vp],
        "q4b_chain_trace_read": [vp, vp, u64, P(u32), P(u32), vp, u32],
        "q4b_chain_run": [vp, vp, P(u32), P(C.c_float)],
        "q4b_chain_set_spin_limit": [vp, u32],
        "q4b_chain_phase_count": [vp, P(u32)],
        "q4b_matvec_noalloc": [i32, vp, u64, vp, vp, vp, u64, vp, vp],
        "q4b_shard_free": [vp, u32],
        "q4b_store_open": [C.c_char_p, P(vp)],
        "q4b_store_tensor_count": [vp, P(u64)],
        "q4b_store_shard_count": [vp, P(u64)],
        "q4b_store_mapped_bytes": [vp, P(u64)],
        "q4b_store_indexed_tensor_bytes": [vp, P(u64)],
        "q4b_store_quantized_groups": [vp, P(u64)],
        "q4b_store_tensor": [vp, C.c_char_p, P(TensorInfo)],
        "q4b_store_tensor_name": [vp, u64, P(C.c_char_p)],
        "q4b_store_tensor_data": [vp, C.c_char_p, P(vp), P(u64)],
        "q4b_store_shard_data": [vp, u64, P(vp), P(u64)],
        "q4b_store_tensor_values_f32": [vp, C.c_char_p, vp, u64, P(u64)],
        "q4b_store_q4_matrix": [vp, C.c_char_p, P(Q4Matrix)],
        "q4b_q4_matrix_from_tensors": [C.c_char_p, P(TensorInfo), P(TensorInfo), P(TensorInfo), P(Q4Matrix)],
        "q4b_weights_open": [vp, C.c_char_p, P(vp)],
        "q4b_weights_open_sharded": [vp, C.c_char_p, u32, u32, P(vp)],
        "q4b_weights_store": [vp, P(vp)],
        "q4b_weights_shard_count": [vp, P(u64)],
        "q4b_weights_device_bytes": [vp, P(u64)],
        "q4b_weights_q4_matrix": [vp, C.c_char_p, P(Q4Matrix)],
        "q4b_weights_jobs": [vp, P(Q4Matrix), u32, u64, P(Job)],
        "q4b_weights_matvec_batch": [vp, P(Q4Matrix), u32, vp, u64, P(vp)],
        "q4b_weights_matmul_batch": [vp, P(Q4Matrix), u32, vp, u64, u64, P(vp)],
        "q4b_weights_argmax_batch": [vp, P(Q4Matrix), vp, u64, u64, vp],
        "q4b_weights_mlp_batch": [vp, P(Q4Matrix), P(Q4Matrix), P(Q4Matrix), vp, u64, u64, vp],
        "q4b_weights_dequantized_row": [vp, P(Q4Matrix), u64, vp],
    }
    for name, argtypes in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int
    lib.q4b_runtime_destroy.argtypes = [vp]
    lib.q4b_runtime_destroy.restype = None
    lib.q4b_last_error.argtypes = []
    lib.q4b_last_error.restype = C.c_char_p
    for name in ("q4b_store_close", "q4b_weights_close"):
        getattr(lib, name).argtypes = [vp]
        getattr(lib, name).restype = None
    lib.q4b_chain_destroy.argtypes = [vp]
    lib.q4b_chain_destroy.restype = None
    lib.q4b_chain_max_k.argtypes = []
    lib.q4b_chain_max_k.restype = C.c_uint64
    lib.q4b_noalloc_last_error.argtypes = []
    lib.q4b_noalloc_last_error.restype = C.c_char_p
    lib.q4b_status_name.argtypes = [i32]
    lib.q4b_status_name.restype = C.c_char_p
    _lib = lib
    return lib


EXPORTS = [
    "q4b_runtime_create", "q4b_runtime_destroy", "q4b_last_error", "q4b_status_name", "q4b_device_info",
    "q4b_shard_upload", "q4b_shard_alloc", "q4b_shard_write", "q4b_shard_read", "q4b_shard_count",
    "q4b_shard_info", "q4b_offset_is_aligned", "q4b_matvec_batch", "q4b_matmul_batch", "q4b_argmax_batch",
    "q4b_mlp_batch", "q4b_mlp_batch_device", "q4b_matmul_add_batch", "q4b_dequantize_row", "q4b_matmul_batch_device",
    "q4b_argmax_batch_device", "q4b_swiglu_device", "q4b_rms_unit_bf16_device", "q4b_synth_q4_device",
    "q4b_synth_bf16_device", "q4b_describe_dispatch", "q4b_launch_count", "q4b_profile_begin", "q4b_profile_end", "q4b_trace_enable", "q4b_trace_read", "q4b_device_status", "q4b_matvec_noalloc", "q4b_noalloc_last_error", "q4b_chain_create", "q4b_chain_run_device", "q4b_chain_run",
    "q4b_chain_set_spin_limit", "q4b_chain_phase_count", "q4b_chain_destroy", "q4b_chain_max_k", "q4b_chain_trace_read", "q4b_arena_create", "q4b_arena_open",
    "q4b_shard_free",
]

# include/q4b_weights.h
WEIGHTS_EXPORTS = [
    "q4b_store_open", "q4b_store_close", "q4b_store_tensor_count", "q4b_store_shard_count", "q4b_store_mapped_bytes",
    "q4b_store_indexed_tensor_bytes", "q4b_store_quantized_groups", "q4b_store_tensor", "q4b_store_tensor_name",
    "q4b_store_tensor_data", "q4b_store_shard_data", "q4b_store_tensor_values_f32", "q4b_store_q4_matrix",
    "q4b_q4_matrix_from_tensors", "q4b_weights_open", "q4b_weights_open_sharded", "q4b_weights_close",
    "q4b_weights_store", "q4b_weights_shard_count", "q4b_weights_device_bytes", "q4b_weights_q4_matrix",
    "q4b_weights_jobs", "q4b_weights_matvec_batch", "q4b_weights_matmul_batch", "q4b_weights_argmax_batch",
    "q4b_weights_mlp_batch", "q4b_weights_dequantized_row",
]
