"""q4-probe: time one grouped Q4 projection launch (the twin of the reference's `q4-probe`
subcommand, src/main.rs:100-150, which times `q4_affine_matvec` / `q4_affine_matmul_batch` on one tensor).

    python -m qwen38_metal_b200.probe --k 5120 --rows 17408,17408 --batch 1 --iterations 20

Weights are synthetic (seeded, generated in HBM) instead of a checkpoint tensor; `--copies` distinct
copies of the weight set are cycled so that consecutive launches stream from HBM, not from L2.
The input follows the reference's probe: x[i] = ((i % 29) - 14) / 29. Two timings are printed: the
device-resident launch (CUDA events on the launching stream) and, with `--host`, the host-buffer entry
point the reference's probe times (upload, launch, download, synchronise).
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--rows", default="5120", help="comma-separated output rows, one projection each (grouped launch)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iterations", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--offset", type=int, default=0, help="byte offset of every tensor from a 16-byte boundary")
    ap.add_argument("--copies", type=int, default=0, help="distinct weight copies to cycle (0: enough to exceed 2x L2)")
    ap.add_argument("--host", action="store_true", help="also time the host-buffer entry point")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--seed", type=int, default=20260)
    args = ap.parse_args()

    import torch

    from . import capi
    from .runtime import CudaRuntime, MappedQ4AffineJob
    from .stack import weight_bytes

    rows = [int(r) for r in args.rows.split(",")]
    k, m = args.k, args.batch
    set_bytes = sum(weight_bytes(n, k) for n in rows)
    copies = args.copies or max(1, int(np.ceil(2 * 126e6 / set_bytes)))
    torch.cuda.set_device(args.device)
    rt = CudaRuntime(args.device)
    sets = []
    for c in range(copies):
        jobs = []
        for i, n in enumerate(rows):
            off = args.offset
            wb = rt.alloc_shard(n * (k // 2) + off)
            sb = rt.alloc_shard(n * (k // 64) * 2 + off)
            bb = rt.alloc_shard(n * (k // 64) * 2 + off)
            job = MappedQ4AffineJob(wb, off, sb, off, bb, off, n, off % 4 == 0)
            rt.synth_q4(args.seed, c * 100 + i, 0.02, 0, n, k, job)
            jobs.append(job)
        sets.append(jobs)
    idx = np.arange(m * k)
    x32 = (((idx % 29).astype(np.float32) - 14.0) / 29.0).astype(np.float32)
    if args.dtype == "bf16":
        xt = torch.from_numpy(x32).to(torch.bfloat16).cuda()
        dtype = capi.Q4B_BF16
    else:
        xt = torch.from_numpy(x32).cuda()
        dtype = capi.Q4B_F32
    outs = [torch.zeros(m * n, dtype=torch.float32, device="cuda") for n in rows]
    ptrs = [o.data_ptr() for o in outs]
    stream = torch.cuda.current_stream()
    print("dispatch:", rt.describe_dispatch(dtype, m, k, sets[0]))
    for i in range(args.warmup):
        rt.matmul_batch_device(xt.data_ptr(), dtype, m, k, sets[i % copies], ptrs, 0, stream.cuda_stream)
    torch.cuda.synchronize()
    rt.profile_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(args.iterations):
        rt.matmul_batch_device(xt.data_ptr(), dtype, m, k, sets[i % copies], ptrs, 0, stream.cuda_stream)
    e1.record(stream)
    torch.cuda.synchronize()
    prof = rt.profile_end()
    ms = e0.elapsed_time(e1) / args.iterations
    kernel_us = prof["ms"] * 1e3 / max(1, prof["launches"])
    checksum = float(sum(o.double().sum().item() for o in outs))
    result = {
        "execution": "CUDA sm_100a Q4 affine projection", "k": k, "rows": rows, "batch": m, "dtype": args.dtype,
        "offset": args.offset, "copies": copies, "iterations": args.iterations,
        "weight_bytes_per_launch": set_bytes, "ms_per_call_device": ms,
        "gbs_per_call_device": set_bytes / (ms * 1e-3) / 1e9,
        "kernel_us": kernel_us, "kernel_gbs": prof["bytes"] / max(1, prof["launches"]) / (kernel_us * 1e-6) / 1e9,
        "tflops": 2.0 * m * sum(rows) * k / (kernel_us * 1e-6) / 1e12,
        "output_checksum": checksum,
    }
    if args.host:
        xh = x32 if args.dtype == "f32" else (x32.view(np.uint32) >> 16).astype(np.uint16)
        if args.dtype == "bf16":
            xh = xt.view(torch.int16).cpu().numpy().view(np.uint16)
        t0 = time.perf_counter()
        for i in range(args.iterations):
            if m == 1:
                rt.q4_affine_matvec_mapped_batch(xh, sets[i % copies])
            else:
                rt.q4_affine_matmul_mapped_batch(xh, m, sets[i % copies])
        result["ms_per_call_host"] = (time.perf_counter() - t0) * 1e3 / args.iterations
    print(json.dumps(result))
    rt.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
