"""Row sharding of the projection stack over two ranks, on CPU with the gloo backend.

Each rank generates only its own rows of every projection (the generator is row-addressable), computes its
slice with the CPU oracle, and the slices are gathered with the same helpers the GPU benchmark uses
(`gather_rows`, `pick_token`). The gathered result must equal the unsharded one bit for bit: a row's sum does not
depend on which rank owns it."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, rows, k: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import q4_oracle as oracle
        from qwen38_metal_b200.stack import gather_rows, pick_token, shard_rows

        x = oracle.bf16_to_f32(oracle.synth_bf16(5, 999, k))
        outs = []
        for tensor, n in enumerate(rows):
            r0, r1 = shard_rows(n, rank, world)
            full = torch.zeros(n, dtype=torch.float32)
            if r1 > r0:
                w, s, b = oracle.synth_q4(5, tensor, r1 - r0, k, row0=r0)
                full[r0:r1] = torch.from_numpy(oracle.matmul_factored_f32(x, w, s, b, r1 - r0)[0])
            gather_rows(dist, full, n, rank, world)
            outs.append(full.numpy().copy())
        # lm_head style exchange: each rank's best (value, id) over its slice of the last projection
        n = rows[-1]
        r0, r1 = shard_rows(n, rank, world)
        pairs = torch.zeros(world, 2, dtype=torch.float32)
        if r1 > r0:
            local = outs[-1][r0:r1]
            pairs[rank, 0] = float(local.max())
            pairs[rank, 1] = float(r0 + int(np.argmax(local)))
        else:
            pairs[rank, 0] = float("-inf")
        gathered = [torch.zeros(2) for _ in range(world)]
        dist.all_gather(gathered, pairs[rank].clone())
        token = int(pick_token(torch.stack(gathered)).item())
        if rank == 0:
            results["outs"] = outs
            results["token"] = token
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows", [(64, 48, 16), (33, 5, 1)])
def test_two_rank_row_sharding_equals_unsharded(rows, oracle):
    k, world = 256, 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), rows, k, results), nprocs=world, join=True)
    x = oracle.bf16_to_f32(oracle.synth_bf16(5, 999, k))
    for tensor, n in enumerate(rows):
        w, s, b = oracle.synth_q4(5, tensor, n, k)
        whole = oracle.matmul_factored_f32(x, w, s, b, n)[0]
        assert np.array_equal(results["outs"][tensor], whole)
    assert results["token"] == int(oracle.argmax_rows(results["outs"][-1][None, :])[0])


def test_shard_rows_cover_every_row_once():
    from qwen38_metal_b200.stack import shard_rows

    for n in (1, 5, 48, 1000, 248320):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_rows(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def test_pick_token_prefers_lowest_id_on_ties():
    from qwen38_metal_b200.stack import pick_token

    pairs = torch.tensor([[1.5, 7.0], [2.5, 300.0], [2.5, 120.0], [0.0, 2.0]])
    assert int(pick_token(pairs).item()) == 120
