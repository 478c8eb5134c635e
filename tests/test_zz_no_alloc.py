"""q4b_matvec_noalloc: the entry point for callers that may not allocate device memory (they are handed
pointers and a stream, or run where cudaMalloc is forbidden). Its scratch is a static device array, so the test
checks what such a caller relies on: the same numbers as the regular entry point, twice in a row (the array keeps
the previous call's contents), for aligned and byte-offset tensors, and a clear refusal past the size limit.
This file sorts last on purpose: a run that stops at the first failure has then run every other test."""
import ctypes as C

import numpy as np
import pytest

from helpers import upload_matrix

pytestmark = pytest.mark.gpu


def _device_array(rt, data):
    buf = rt.buffer_from_slice(data)
    return buf, rt.shard_pointer(buf)


@pytest.mark.parametrize("n,k,offset", [(1000, 5120, 0), (333, 1024, 0), (77, 640, 2), (48, 17408, 0)])
def test_noalloc_matches_regular_entry_point_twice(runtime, oracle, n, k, offset):
    from qwen38_metal_b200 import capi

    lib = capi.load()
    w, s, b = oracle.synth_q4(909, n, n, k)
    job = upload_matrix(runtime, w, s, b, offset=offset)
    x_bits = oracle.synth_bf16(909, 5000 + k, k)
    expected = runtime.q4_affine_matvec_mapped_batch(x_bits, [job])[0]
    xbuf, xptr = _device_array(runtime, x_bits)
    obuf = runtime.alloc_shard(n * 4)
    optr = runtime.shard_pointer(obuf)
    wp = runtime.shard_pointer(job.weights) + job.weight_offset
    sp = runtime.shard_pointer(job.scales) + job.scale_offset
    bp = runtime.shard_pointer(job.biases) + job.bias_offset
    for _ in range(2):
        runtime.write_shard(obuf, 0, np.full(n, np.nan, dtype=np.float32))
        st = lib.q4b_matvec_noalloc(0, xptr, k, wp, sp, bp, n, optr, None)
        assert st == 0, lib.q4b_noalloc_last_error()
        got = runtime.read_shard(obuf, 0, n * 4).view(np.float32)  # read_shard synchronises the device
        # same kernel, possibly a different split of tiles between warps: fp32 sums may differ in the last bits
        assert oracle.rel_l2(got, expected) <= 1e-6
        x = oracle.bf16_to_f32(x_bits)
        assert oracle.rel_l2(got, oracle.matmul_factored_f32(x, w, s, b, n)[0]) <= 1e-5


def test_noalloc_rejects_what_the_static_array_cannot_hold(runtime):
    from qwen38_metal_b200 import capi

    lib = capi.load()
    buf = runtime.alloc_shard(4096)
    p = runtime.shard_pointer(buf)
    assert lib.q4b_matvec_noalloc(0, p, 32768 + 64, p, p, p, 16, p, None) == 14  # Unsupported
    assert b"32768" in lib.q4b_noalloc_last_error()
    assert lib.q4b_matvec_noalloc(0, p, 100, p, p, p, 16, p, None) == 5          # InputNotGrouped
    assert lib.q4b_matvec_noalloc(0, None, 128, p, p, p, 16, p, None) == 13       # InvalidArgument


@pytest.mark.parametrize("n,k,offset", [(40, 192, 0), (33, 192, 2), (50, 1024, 6), (16, 5120, 0)])
def test_noalloc_on_tensors_without_padding(runtime, oracle, n, k, offset):
    """Callers of this entry point bring their own tensors, which nothing pads: the three arrays here are torch byte
    buffers of exactly offset + size bytes (the library's own shards carry 1 KB of slack, these do not), with an odd
    group count and byte offsets in the mix. The kernels read only 16-byte blocks that a tensor itself touches (the
    address arithmetic is checked on the CPU in tests/test_decomp.py); here the results must match the oracle."""
    import torch

    from qwen38_metal_b200 import capi

    lib = capi.load()
    w, s, b = oracle.synth_q4(910, n + k, n, k)
    x_bits = oracle.synth_bf16(910, 6000 + k, k)

    def exact(arr):
        raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
        buf = torch.zeros(offset + raw.size, dtype=torch.uint8, device="cuda")
        buf[offset:] = torch.from_numpy(raw.copy()).cuda()
        return buf

    wb, sb, bb = exact(w), exact(s), exact(b)
    xb = torch.from_numpy(x_bits.view(np.int16).copy()).cuda()
    out = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    for _ in range(2):
        st = lib.q4b_matvec_noalloc(0, xb.data_ptr(), k, wb.data_ptr() + offset, sb.data_ptr() + offset, bb.data_ptr() + offset, n,
                                    out.data_ptr(), None)
        assert st == 0, lib.q4b_noalloc_last_error()
        torch.cuda.synchronize()
        x = oracle.bf16_to_f32(x_bits)
        assert oracle.rel_l2(out.cpu().numpy(), oracle.matmul_factored_f32(x, w, s, b, n)[0]) <= 1e-5
