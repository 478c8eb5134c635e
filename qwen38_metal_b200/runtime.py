"""Python mirror of the reference's Q4 runtime interface, over the C ABI.

Names and argument meaning follow `MetalRuntime` and `MappedQ4AffineJob` of the reference
(src/metal_runtime.rs:79-192, 929-982, 3523-3891, 4479-4689) so tests read like the
reference's own: `runtime.q4_affine_matvec_mapped_batch(input, [MappedQ4AffineJob(...)])`.
Every call goes through `lib/libq4b200.so`; there is no fallback.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import capi


class Q4RuntimeError(RuntimeError):
    """MetalRuntimeError of the reference (src/metal_runtime.rs:9218-9257); `.kind` is the variant name."""

    def __init__(self, status: int, message: str):
        self.status = status
        self.kind = capi.STATUS_NAMES.get(status, "Unknown")
        super().__init__(f"{self.kind}: {message}")


def _check(status: int) -> None:
    if status != 0:
        raise Q4RuntimeError(status, capi.load().q4b_last_error().decode("utf-8", "replace"))


@dataclass(frozen=True)
class DeviceBuffer:
    """A weight shard resident in HBM (the reference's `metal::Buffer`)."""

    shard: int
    length: int


@dataclass(frozen=True)
class MappedQ4AffineJob:
    """MappedQ4AffineJob::new, src/metal_runtime.rs:171-191 -- same argument order."""

    weights: DeviceBuffer
    weight_offset: int
    scales: DeviceBuffer
    scale_offset: int
    biases: DeviceBuffer
    bias_offset: int
    output_rows: int
    aligned: bool = True

    def to_c(self) -> capi.Job:
        return capi.Job(self.weights.shard, self.scales.shard, self.biases.shard, 1 if self.aligned else 0,
                        self.weight_offset, self.scale_offset, self.bias_offset, self.output_rows)


def _activation(x) -> tuple[np.ndarray, int]:
    """fp32 arrays are the reference's activation type; uint16 arrays are taken as bf16 bits."""
    x = np.ascontiguousarray(x)
    if x.dtype == np.uint16:
        return x, capi.Q4B_BF16
    return np.ascontiguousarray(x, dtype=np.float32), capi.Q4B_F32


def _jobs(jobs) -> "C.Array":
    arr = (capi.Job * len(jobs))()
    for i, j in enumerate(jobs):
        arr[i] = j.to_c()
    return arr


class CudaRuntime:
    """The B200 stand-in for `MetalRuntime` (Q4 projection part)."""

    def __init__(self, device: int = 0):
        self._lib = capi.load()
        handle = C.c_void_p()
        _check(self._lib.q4b_runtime_create(device, C.byref(handle)))
        self._h = handle
        self.device = device

    # -- lifetime ------------------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.q4b_runtime_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    def device_info(self) -> dict:
        sm, total, name = C.c_int(), C.c_uint64(), C.create_string_buffer(128)
        _check(self._lib.q4b_device_info(self._h, C.byref(sm), C.byref(total), name, 128))
        return {"sm_count": sm.value, "total_bytes": total.value, "name": name.value.decode()}

    # -- shards --------------------------------------------------------------------------
    def buffer_from_slice(self, data) -> DeviceBuffer:
        """MetalRuntime::buffer_from_slice: upload bytes verbatim."""
        data = np.ascontiguousarray(data)
        raw = data.view(np.uint8).reshape(-1)
        shard = C.c_uint32()
        _check(self._lib.q4b_shard_upload(self._h, raw.ctypes.data_as(C.c_void_p), raw.size, C.byref(shard)))
        return DeviceBuffer(shard.value, raw.size)

    def alloc_shard(self, nbytes: int) -> DeviceBuffer:
        shard = C.c_uint32()
        _check(self._lib.q4b_shard_alloc(self._h, nbytes, C.byref(shard)))
        return DeviceBuffer(shard.value, nbytes)

    def write_shard(self, buf: DeviceBuffer, offset: int, data) -> None:
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        _check(self._lib.q4b_shard_write(self._h, buf.shard, offset, raw.ctypes.data_as(C.c_void_p), raw.size))

    def read_shard(self, buf: DeviceBuffer, offset: int, nbytes: int) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        _check(self._lib.q4b_shard_read(self._h, buf.shard, offset, out.ctypes.data_as(C.c_void_p), nbytes))
        return out

    def shard_count(self) -> int:
        n = C.c_uint32()
        _check(self._lib.q4b_shard_count(self._h, C.byref(n)))
        return n.value

    def shard_pointer(self, buf: DeviceBuffer) -> int:
        p, n = C.c_void_p(), C.c_uint64()
        _check(self._lib.q4b_shard_info(self._h, buf.shard, C.byref(p), C.byref(n)))
        return p.value

    def offset_is_aligned(self, buf: DeviceBuffer, offset: int, alignment: int) -> bool:
        out = C.c_int()
        _check(self._lib.q4b_offset_is_aligned(self._h, buf.shard, offset, alignment, C.byref(out)))
        return bool(out.value)

    # -- host-buffer projections ------------------------------------------------------------
    def q4_affine_matvec(self, input, packed_weights, scales, biases, output_rows: int) -> np.ndarray:
        """MetalRuntime::q4_affine_matvec, src/metal_runtime.rs:929-953: slices in, aligned matvec."""
        x, _ = _activation(input)
        w = np.ascontiguousarray(packed_weights, dtype=np.uint32).reshape(-1)
        s = np.ascontiguousarray(scales, dtype=np.uint16).reshape(-1)
        b = np.ascontiguousarray(biases, dtype=np.uint16).reshape(-1)
        # MatvecShape::validate, src/metal_runtime.rs:8933-8983
        if x.size == 0 or output_rows == 0:
            raise Q4RuntimeError(4, "matrix dimensions must be greater than zero")
        if x.size % 64 != 0:
            raise Q4RuntimeError(5, f"input dimension {x.size} is not divisible by affine group size 64")
        for name, arr, expected in (("packed_weights", w, output_rows * (x.size // 8)),
                                    ("scales", s, output_rows * (x.size // 64)),
                                    ("biases", b, output_rows * (x.size // 64))):
            if arr.size != expected:
                raise Q4RuntimeError(6, f"{name} has {arr.size} elements, expected {expected}")
        job = MappedQ4AffineJob(self.buffer_from_slice(w), 0, self.buffer_from_slice(s), 0,
                                self.buffer_from_slice(b), 0, output_rows, True)
        return self.q4_affine_matvec_mapped_batch(x, [job])[0]

    def q4_affine_matvec_mapped_batch(self, input, jobs) -> list[np.ndarray]:
        """src/metal_runtime.rs:3599-3678: several projections over one activation."""
        x, dtype = _activation(input)
        outs = [np.empty(max(int(j.output_rows), 0), dtype=np.float32) for j in jobs]
        ptrs = (C.c_void_p * max(len(jobs), 1))(*[o.ctypes.data for o in outs])
        _check(self._lib.q4b_matvec_batch(self._h, x.ctypes.data_as(C.c_void_p), dtype, x.size, _jobs(jobs),
                                          len(jobs), ptrs))
        return outs

    def q4_affine_matmul_mapped_batch(self, input, batch_size: int, jobs) -> list[np.ndarray]:
        """src/metal_runtime.rs:3683-3792: row-major [batch][rows] per job."""
        x, dtype = _activation(input)
        if not jobs or batch_size == 0 or x.size == 0 or x.size % batch_size != 0:
            raise Q4RuntimeError(4, "matrix dimensions must be greater than zero")
        k = x.size // batch_size
        outs = [np.empty((batch_size, int(j.output_rows)), dtype=np.float32) for j in jobs]
        ptrs = (C.c_void_p * len(jobs))(*[o.ctypes.data for o in outs])
        _check(self._lib.q4b_matmul_batch(self._h, x.ctypes.data_as(C.c_void_p), dtype, batch_size, k, _jobs(jobs),
                                          len(jobs), ptrs))
        return outs

    def q4_affine_matmul_add_mapped_batch(self, input, batch_size: int, jobs, residuals) -> list[np.ndarray]:
        """encode_q4_affine_matmul_add, src/metal_runtime.rs:5644-5798: residual += projection."""
        x, dtype = _activation(input)
        k = x.size // batch_size
        outs = [np.array(r, dtype=np.float32, copy=True).reshape(batch_size, int(j.output_rows))
                for r, j in zip(residuals, jobs)]
        ptrs = (C.c_void_p * len(jobs))(*[o.ctypes.data for o in outs])
        _check(self._lib.q4b_matmul_add_batch(self._h, x.ctypes.data_as(C.c_void_p), dtype, batch_size, k,
                                              _jobs(jobs), len(jobs), ptrs))
        return outs

    def q4_affine_argmax_mapped_batch(self, input, batch_size: int, job) -> np.ndarray:
        """src/metal_runtime.rs:3797-3891."""
        x, dtype = _activation(input)
        if batch_size == 0 or x.size == 0 or x.size % batch_size != 0:
            raise Q4RuntimeError(4, "matrix dimensions must be greater than zero")
        tokens = np.empty(batch_size, dtype=np.uint32)
        cj = job.to_c()
        _check(self._lib.q4b_argmax_batch(self._h, x.ctypes.data_as(C.c_void_p), dtype, batch_size,
                                          x.size // batch_size, C.byref(cj), tokens.ctypes.data_as(C.c_void_p)))
        return tokens

    def q4_affine_mlp_mapped_batch(self, input, batch_size: int, gate, up, down) -> np.ndarray:
        """src/metal_runtime.rs:4479-4689."""
        x, dtype = _activation(input)
        if batch_size == 0 or x.size == 0 or x.size % batch_size != 0:
            raise Q4RuntimeError(4, "matrix dimensions must be greater than zero")
        out = np.empty((batch_size, int(down.output_rows)), dtype=np.float32)
        g, u, d = gate.to_c(), up.to_c(), down.to_c()
        _check(self._lib.q4b_mlp_batch(self._h, x.ctypes.data_as(C.c_void_p), dtype, batch_size, x.size // batch_size,
                                       C.byref(g), C.byref(u), C.byref(d), out.ctypes.data_as(C.c_void_p)))
        return out

    def dequantized_row(self, job, k: int, row: int) -> np.ndarray:
        """dequantized_row, src/native.rs:4944-4987."""
        out = np.empty(k, dtype=np.float32)
        cj = job.to_c()
        _check(self._lib.q4b_dequantize_row(self._h, C.byref(cj), k, row, out.ctypes.data_as(C.c_void_p)))
        return out

    # -- device-resident twins (raw device pointers as ints) -----------------------------------
    def matmul_batch_device(self, x_ptr: int, dtype: int, m: int, k: int, jobs, out_ptrs, flags: int = 0,
                            stream: int = 0) -> None:
        ptrs = (C.c_void_p * len(jobs))(*out_ptrs)
        _check(self._lib.q4b_matmul_batch_device(self._h, x_ptr, dtype, m, k, _jobs(jobs), len(jobs), ptrs, flags,
                                                 stream))

    def mlp_batch_device(self, x_ptr: int, dtype: int, m: int, k: int, gate, up, down, out_ptr: int, stream: int = 0) -> None:
        g, u, d = gate.to_c(), up.to_c(), down.to_c()
        _check(self._lib.q4b_mlp_batch_device(self._h, x_ptr, dtype, m, k, C.byref(g), C.byref(u), C.byref(d), out_ptr, stream))

    def argmax_batch_device(self, x_ptr: int, dtype: int, m: int, k: int, job, index_base: int, tokens_ptr: int,
                            values_ptr: int = 0, stream: int = 0) -> None:
        cj = job.to_c()
        _check(self._lib.q4b_argmax_batch_device(self._h, x_ptr, dtype, m, k, C.byref(cj), index_base, tokens_ptr,
                                                 values_ptr or None, stream))

    def swiglu_device(self, gate_ptr: int, up_ptr: int, count: int, out_f32_ptr: int = 0, out_bf16_ptr: int = 0,
                      stream: int = 0) -> None:
        _check(self._lib.q4b_swiglu_device(self._h, gate_ptr, up_ptr, count, out_f32_ptr or None,
                                           out_bf16_ptr or None, stream))

    def rms_unit_bf16_device(self, in_ptr: int, rows: int, n: int, eps: float, out_ptr: int, stream: int = 0) -> None:
        _check(self._lib.q4b_rms_unit_bf16_device(self._h, in_ptr, rows, n, eps, out_ptr, stream))

    # -- persistent decode chain ----------------------------------------------------------------------
    def arena_create(self, nbytes: int) -> tuple[int, bytes]:
        """Zeroed device memory that peer processes can map: (device pointer, 64-byte IPC handle)."""
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        _check(self._lib.q4b_arena_create(self._h, nbytes, C.byref(ptr), handle))
        return ptr.value, handle.raw

    def arena_open(self, handle: bytes) -> int:
        ptr = C.c_void_p()
        _check(self._lib.q4b_arena_open(self._h, handle, C.byref(ptr)))
        return ptr.value

    def chain_create(self, stages, logits_ptr: int = 0, vocab: int = 0, index_base: int = 0, token_ptr: int = 0,
                     best_ptr: int = 0, peers=None) -> "DecodeChain":
        """stages: list of dicts {x_kind, k, src0, src1, x_bf16_out, jobs, outputs, eps[, peer_outputs, k_total,
        k_begin, src_parts, src_part_stride, sum_out]} with raw device pointers (see q4b_stage);
        peers: None or {world, rank, flags: [ptr]*world, cand: [ptr]*world}."""
        arr = (capi.Stage * len(stages))()
        keep = []
        for i, s in enumerate(stages):
            jobs = _jobs(s["jobs"])
            outs = (C.c_void_p * len(s["jobs"]))(*s["outputs"])
            keep += [jobs, outs]
            mirrors = None
            if s.get("peer_outputs") is not None:
                flat = [p or None for row in s["peer_outputs"] for p in (list(row) + [0] * 8)[:8]]
                mirrors = (C.c_void_p * len(flat))(*flat)
                keep.append(mirrors)
            arr[i] = capi.Stage(s["x_kind"], s.get("eps", 1e-6), s["k"], s["src0"], s.get("src1") or None,
                                s.get("x_bf16_out") or None, jobs, len(s["jobs"]), outs, mirrors,
                                s.get("k_total", 0), s.get("k_begin", 0), s.get("src_parts", 0), 0,
                                s.get("src_part_stride", 0), s.get("sum_out") or None)
        cpeers = None
        if peers is not None:
            cpeers = capi.Peers(peers["world"], peers["rank"])
            for r in range(peers["world"]):
                cpeers.flags[r] = peers["flags"][r]
                cpeers.cand[r] = peers["cand"][r]
        handle = C.c_void_p()
        _check(self._lib.q4b_chain_create(self._h, arr, len(stages), logits_ptr or None, vocab, index_base,
                                          token_ptr or None, best_ptr or None,
                                          C.byref(cpeers) if cpeers is not None else None, C.byref(handle)))
        return DecodeChain(self, handle)

    # -- synthetic tensors ---------------------------------------------------------------------
    def synth_q4(self, seed: int, tensor: int, sigma: float, row0: int, rows: int, k: int, job) -> None:
        cj = job.to_c()
        _check(self._lib.q4b_synth_q4_device(self._h, seed, tensor, sigma, row0, rows, k, C.byref(cj)))

    def synth_bf16(self, seed: int, tensor: int, count: int, out_ptr: int, stream: int = 0) -> None:
        _check(self._lib.q4b_synth_bf16_device(self._h, seed, tensor, count, out_ptr, stream))

    # -- introspection ---------------------------------------------------------------------------
    def describe_dispatch(self, dtype: int, m: int, k: int, jobs) -> str:
        buf = C.create_string_buffer(256)
        _check(self._lib.q4b_describe_dispatch(self._h, dtype, m, k, _jobs(jobs), len(jobs), buf, 256))
        return buf.value.decode()

    def profile_begin(self) -> None:
        _check(self._lib.q4b_profile_begin(self._h))

    def profile_end(self) -> dict:
        """Timed projection-kernel launches since profile_begin: count, summed ms, algorithmic bytes."""
        n, ms, nbytes, flops = C.c_uint64(), C.c_double(), C.c_uint64(), C.c_uint64()
        _check(self._lib.q4b_profile_end(self._h, C.byref(n), C.byref(ms), C.byref(nbytes), C.byref(flops)))
        return {"launches": n.value, "ms": ms.value, "bytes": nbytes.value, "flops": flops.value}

    def trace_enable(self, on: bool = True) -> None:
        _check(self._lib.q4b_trace_enable(self._h, 1 if on else 0))

    def device_status(self) -> None:
        """Synchronise and raise if a device-resident call failed asynchronously."""
        _check(self._lib.q4b_device_status(self._h))

    def launch_count(self) -> int:
        n = C.c_uint64()
        _check(self._lib.q4b_launch_count(self._h, C.byref(n)))
        return n.value


class DecodeChain:
    """A compiled list of stages run by one cooperative kernel launch (`q4b_chain_*`)."""

    def __init__(self, rt: CudaRuntime, handle):
        self._rt, self._h = rt, handle

    def run(self, stream: int = 0) -> None:
        _check(self._rt._lib.q4b_chain_run_device(self._h, stream))

    def run_host(self, x_bits) -> tuple[int, float]:
        """Host slice in, token out (q4b_chain_run): x_bits is the first stage's bf16 activation as uint16 (a numpy
        array, or an integer address of k pinned uint16 values). Returns (token id, winning logit)."""
        token, best = C.c_uint32(), C.c_float()
        ptr = x_bits if isinstance(x_bits, int) else np.ascontiguousarray(x_bits, dtype=np.uint16).ctypes.data
        _check(self._rt._lib.q4b_chain_run(self._h, ptr, C.byref(token), C.byref(best)))
        return token.value, best.value

    def set_spin_limit(self, polls: int) -> None:
        _check(self._rt._lib.q4b_chain_set_spin_limit(self._h, polls))

    def phase_count(self) -> int:
        n = C.c_uint32()
        _check(self._rt._lib.q4b_chain_phase_count(self._h, C.byref(n)))
        return n.value

    def trace_read(self):
        """(stamps [blocks][phases][16] uint64 ns, phase_info [phases]) of the last run; the chain must have been
        created after CudaRuntime.trace_enable(True)."""
        phases = self.phase_count()
        sms = self._rt.device_info()["sm_count"]
        stamps = np.zeros(sms * phases * 16, dtype=np.uint64)
        info = np.zeros(phases, dtype=np.uint32)
        nb, nph = C.c_uint32(), C.c_uint32()
        _check(self._rt._lib.q4b_chain_trace_read(self._h, stamps.ctypes.data_as(C.c_void_p), stamps.size, C.byref(nb),
                                                  C.byref(nph), info.ctypes.data_as(C.c_void_p), phases))
        return stamps.reshape(nb.value, nph.value, 16), info

    def close(self) -> None:
        if self._h:
            self._rt._lib.q4b_chain_destroy(self._h)
            self._h = None
