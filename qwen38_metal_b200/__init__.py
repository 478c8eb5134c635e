"""B200 (sm_100a) implementation of the affine-Q4 projection path of Fuxx-1/qwen38-metal.

All compute lives in `lib/libq4b200.so` (CUDA, built by `qwen38_metal_b200.build`); this package is the
host-side mirror of the reference's projection interface over that library's C ABI
(`include/q4b200.h`). There is no CPU or PyTorch compute path: without the library, or without a
B200, constructing a runtime raises.
"""
from .runtime import CudaRuntime, DeviceBuffer, MappedQ4AffineJob, Q4RuntimeError  # noqa: F401

__all__ = ["CudaRuntime", "DeviceBuffer", "MappedQ4AffineJob", "Q4RuntimeError"]
