"""Shared helpers of the parity tests."""
from __future__ import annotations

import numpy as np

import ref_cases as rc


def golden_rows(case, entry, batch: int, matrix_index: int = 0) -> np.ndarray:
    """Expected [batch][rows] of a fixture; long batches are stored as one period of rows."""
    head = np.asarray(entry["batches"][str(batch)][matrix_index], dtype=np.float64)
    if head.shape[0] == batch:
        return head
    p = case.x[0]
    return head[np.arange(batch) % p]


def upload_matrix(rt, packed, scales, biases, offset: int = 0, rows=None):
    """Upload the three tensors of a projection, each behind `offset` prefix bytes, as the reference's
    unaligned tests do (src/metal_runtime.rs:11944-11960), and return the job."""
    from qwen38_metal_b200.runtime import MappedQ4AffineJob

    packed = np.ascontiguousarray(packed, dtype=np.uint32)
    n = packed.shape[0] if rows is None else rows
    w = rt.buffer_from_slice(rc.prefixed(packed, offset))
    s = rt.buffer_from_slice(rc.prefixed(np.ascontiguousarray(scales, dtype=np.uint16), offset))
    b = rt.buffer_from_slice(rc.prefixed(np.ascontiguousarray(biases, dtype=np.uint16), offset))
    return MappedQ4AffineJob(w, offset, s, offset, b, offset, n, offset % 4 == 0)


def upload_in_one_shard(rt, tensors, start: int, gap_align: int = 1):
    """Lay several (packed, scales, biases) triples into ONE shard beginning at byte `start`, the way a
    safetensors data region does; returns the jobs. `gap_align` pads each tensor start to that multiple."""
    from qwen38_metal_b200.runtime import MappedQ4AffineJob

    blobs, offsets, pos = [], [], start
    for trip in tensors:
        trip_offs = []
        for arr in trip:
            raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
            pad = (-(pos - start)) % gap_align
            if pad:
                blobs.append(np.zeros(pad, dtype=np.uint8))
                pos += pad
            trip_offs.append(pos)
            blobs.append(raw)
            pos += raw.size
        offsets.append(trip_offs)
    image = np.concatenate([np.zeros(start, dtype=np.uint8)] + blobs)
    buf = rt.buffer_from_slice(image)
    jobs = []
    for trip, offs in zip(tensors, offsets):
        jobs.append(MappedQ4AffineJob(buf, offs[0], buf, offs[1], buf, offs[2], trip[0].shape[0], offs[0] % 4 == 0))
    return jobs
