"""Synthetic decode stack: the projection half of the reference's GPU-resident decode graph.

The reference encodes a whole token as one command buffer (`decode_layers`,
src/metal_runtime.rs:2022-2081; per layer `encode_decode_linear_layer` :3301-3520 and
`encode_decode_full_layer` :1567-2020): RMS-norm, three or four projections sharing one activation,
attention/DeltaNet, output projection, RMS-norm, gate/up, SwiGLU, down. Attention and DeltaNet are
not projections and are left out; what remains per layer is

    a (bf16, hidden) -> [q,k,v | qkv,z,b,a | gate,up]  one grouped launch, one activation read
    h = bf16(silu(gate) * up)                          (qwen38_swiglu_rows)
    d = down(h)                                        fp32
    a' = bf16(d / rms(d))                              weightless RMS-norm keeps |a| near 1

and after the last layer lm_head -> argmax. Weights are generated in HBM from a seed
(`CudaRuntime.synth_q4`); every other projection (odd positions of the grouped set, the down projection of odd
layers) starts two bytes off a 16-byte boundary, which is how tensors sit in real safetensors shards. With `world > 1` each rank holds rows
[floor(r*N/W), floor((r+1)*N/W)) of every projection; the caller gathers `h`, `d` and the argmax
candidates between ranks (`gather` callbacks), all other work is local.

torch is used for device buffers, streams and CUDA-graph capture only.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import capi
from .runtime import CudaRuntime, MappedQ4AffineJob

HIDDEN = 5120
INTER = 17408
VOCAB = 248320
# Q/K/V of a full-attention layer and the four DeltaNet input projections, then MLP gate and up
LAYER_ROWS = (6144, 1024, 1024, 6144, 2048, 2048, 48, INTER, INTER)
GATE, UP = 7, 8


def shard_rows(n: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [begin, end) of an n-row projection owned by `rank` (row sharding; may be empty)."""
    return (n * rank) // world, (n * (rank + 1)) // world


def weight_bytes(n: int, k: int) -> int:
    """Packed weights + bf16 scales + bf16 biases of an [n][k] projection: 0.5625 bytes per weight."""
    return n * (k // 2) + 2 * n * (k // 64) * 2


def token_bytes(layers: int = 64, hidden: int = HIDDEN, inter: int = INTER, vocab: int = VOCAB,
                layer_rows=LAYER_ROWS) -> int:
    per_layer = sum(weight_bytes(n, hidden) for n in layer_rows) + weight_bytes(hidden, inter)
    return layers * per_layer + weight_bytes(vocab, hidden)


def gather_rows(dist, tensor, total_rows: int, rank: int, world: int) -> None:
    """Make a row-sharded output whole on every rank, in place: rank r has written rows
    [floor(r*N/W), floor((r+1)*N/W)) of `tensor`. Even splits use one all-gather into the tensor itself;
    uneven splits (N not divisible by W, possibly empty slices) fall back to one broadcast per rank."""
    if world == 1:
        return
    if total_rows % world == 0:
        rows = total_rows // world
        dist.all_gather_into_tensor(tensor[:total_rows], tensor[rank * rows:(rank + 1) * rows])
        return
    for r in range(world):
        r0, r1 = shard_rows(total_rows, r, world)
        if r1 > r0:
            dist.broadcast(tensor[r0:r1], src=r)


def pick_token(pairs):
    """pairs: [world][2] float tensor of (best logit, token id) per vocabulary slice. The winner is the greatest
    logit; equal logits go to the lowest id (shaders/qwen38.metal:4218-4221). Returns a 0-d float tensor."""
    top = pairs[:, 0].max()
    ids = torch.where(pairs[:, 0] == top, pairs[:, 1], torch.full_like(pairs[:, 1], 3.0e38))
    return ids.min()


@dataclass
class Projection:
    job: MappedQ4AffineJob | None  # None when this rank owns no rows
    rows: int                      # rows held here
    row0: int                      # first global row held here
    total_rows: int


class SyntheticStack:
    def __init__(self, rt: CudaRuntime, layers: int = 64, hidden: int = HIDDEN, inter: int = INTER,
                 vocab: int = VOCAB, layer_rows=LAYER_ROWS, seed: int = 20260, rank: int = 0, world: int = 1,
                 misalign: int = 2, device: int = 0):
        self.rt, self.layers, self.hidden, self.inter, self.vocab = rt, layers, hidden, inter, vocab
        self.layer_rows, self.seed, self.rank, self.world = tuple(layer_rows), seed, rank, world
        self.device = torch.device("cuda", device)
        self.misalign = misalign
        self.gate_i, self.up_i = len(layer_rows) - 2, len(layer_rows) - 1
        self.bytes_local = 0
        tensor = 0
        self.proj: list[list[Projection]] = []
        self.down: list[Projection] = []
        for layer in range(layers):
            row = []
            for i, n in enumerate(self.layer_rows):
                row.append(self._make(tensor, n, hidden, misalign if i % 2 else 0))
                tensor += 1
            self.proj.append(row)
            self.down.append(self._make(tensor, hidden, inter, misalign if layer % 2 else 0))
            tensor += 1
        self.lm_head = self._make(tensor, vocab, hidden, 0)
        self.x0_tensor = tensor + 1
        f32, bf16 = torch.float32, torch.bfloat16
        dev = self.device
        # activations (replicated on every rank) and per-rank output slices
        self.x = torch.zeros(hidden, dtype=bf16, device=dev)
        self.outs = [torch.zeros(max(p.total_rows, 1), dtype=f32, device=dev) for p in self.proj[0]]
        self.h = torch.zeros(inter, dtype=bf16, device=dev)
        self.d = torch.zeros(hidden, dtype=f32, device=dev)
        self.token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.best = torch.zeros(1, dtype=f32, device=dev)
        self.checksum = torch.zeros(len(self.layer_rows) - 2, dtype=f32, device=dev)

    def _make(self, tensor: int, n: int, k: int, offset: int, whole: bool = False) -> Projection:
        r0, r1 = (0, n) if whole else shard_rows(n, self.rank, self.world)
        rows = r1 - r0
        if rows == 0:
            return Projection(None, 0, r0, n)
        groups = k // 64
        wb = self.rt.alloc_shard(rows * (k // 2) + offset)
        sb = self.rt.alloc_shard(rows * groups * 2 + offset)
        bb = self.rt.alloc_shard(rows * groups * 2 + offset)
        job = MappedQ4AffineJob(wb, offset, sb, offset, bb, offset, rows, offset % 4 == 0)
        self.rt.synth_q4(self.seed, tensor, 0.02, r0, rows, k, job)
        if not whole:
            self.bytes_local += weight_bytes(rows, k)
        return Projection(job, rows, r0, n)

    def reset_input(self, stream: int = 0) -> None:
        self.rt.synth_bf16(self.seed, self.x0_tensor, self.hidden, self.x.data_ptr(), stream)

    def _grouped(self, x_ptr: int, k: int, projs, outs, stream: int) -> None:
        jobs, ptrs = [], []
        for p, o in zip(projs, outs):
            if p.job is not None:
                jobs.append(p.job)
                ptrs.append(o.data_ptr() + 4 * p.row0)
        if jobs:
            self.rt.matmul_batch_device(x_ptr, capi.Q4B_BF16, 1, k, jobs, ptrs, 0, stream)

    def build_chain(self, layers=None):
        """The whole token as one persistent kernel (single GPU): stage list for `CudaRuntime.chain_create`.
        `layers`: only the first so many layers, then lm_head (shallow chains are what different evaluation orders can
        be compared on: the stack amplifies last-bit differences by about an order of magnitude per layer)."""
        if self.world != 1:
            raise ValueError("the persistent decode chain covers one GPU; sharded stacks use decode_token with gathers")
        stages = []
        gate, up = self.outs[self.gate_i], self.outs[self.up_i]
        for layer in range(self.layers if layers is None else layers):
            projs = self.proj[layer]
            first = layer == 0
            stages.append({"x_kind": capi.X_BF16 if first else capi.X_RMS, "k": self.hidden,
                           "src0": self.x.data_ptr() if first else self.d.data_ptr(), "eps": 1e-6,
                           "x_bf16_out": 0 if first else self.x.data_ptr(),
                           "jobs": [p.job for p in projs], "outputs": [o.data_ptr() for o in self.outs]})
            stages.append({"x_kind": capi.X_SWIGLU, "k": self.inter, "src0": gate.data_ptr(), "src1": up.data_ptr(),
                           "x_bf16_out": self.h.data_ptr(), "jobs": [self.down[layer].job], "outputs": [self.d.data_ptr()]})
        self.logits = torch.zeros(self.vocab, dtype=torch.float32, device=self.device)
        stages.append({"x_kind": capi.X_RMS, "k": self.hidden, "src0": self.d.data_ptr(), "eps": 1e-6,
                       "x_bf16_out": self.x.data_ptr(), "jobs": [self.lm_head.job], "outputs": [self.logits.data_ptr()]})
        return self.rt.chain_create(stages, self.logits.data_ptr(), self.vocab, 0, self.token.data_ptr(),
                                    self.best.data_ptr())

    def sharded_arena_bytes(self) -> int:
        """Size of the exchange arena of `build_chain_sharded`: one partial down output per rank, the barrier words
        and the token candidates."""
        return self.world * ((self.hidden * 16 + 255) & ~255) + 512

    def build_chain_sharded(self, dist, arenas=None, layers=None):
        """The whole token as one persistent kernel per rank. Projections of the hidden activation are row-sharded;
        gate and up are fused into the slice of the SwiGLU vector this rank owns, and the down projection is cut
        along K so that each rank consumes exactly that slice: it multiplies inputs [r0, r1) of the whole down
        matrix (read in place through strided rows) and stores its partial output into every rank's exchange arena
        with peer stores, as tagged words that the next stage's rebuild polls. The next activation is the RMS-norm of
        the partial outputs added in rank order -- no cross-GPU barrier and no collective library on the data path. Summation order differs from the
        single-GPU chain (fp32 partial sums per rank), so results agree to fp32 rounding, not bit for bit.
        `dist` (torch.distributed) only carries the 64-byte IPC handles at set-up. `arenas` (tests): exchange arenas
        already mapped here, one base pointer per rank, in place of the IPC exchange."""
        world, rank, rt = self.world, self.rank, self.rt

        def align(n):
            return (n + 255) & ~255

        # a slot per rank, wide enough for two copies of the partial output as 8-byte {value, tag} words: the chain then
        # hands the partials over without a fence or a cross-GPU barrier (q4b_stage: src_part_stride >= 16 k)
        part_stride = align(self.hidden * 16)
        off_parts, off_flags = 0, world * part_stride
        off_cand = off_flags + 256
        size = off_cand + 256
        assert size == self.sharded_arena_bytes()
        if arenas is None:
            base, handle = rt.arena_create(size)
            handles = [None] * world
            dist.all_gather_object(handles, handle)
            arena = [base if r == rank else rt.arena_open(handles[r]) for r in range(world)]
        else:
            arena, base = list(arenas), arenas[rank]
        self.arena_base = base
        if not hasattr(self, "down_whole"):
            # the whole down matrices (the per-stage path keeps its row slices in self.down)
            first = len(self.layer_rows)
            per_layer = first + 1
            self.down_whole = [self._make(layer * per_layer + first, self.hidden, self.inter,
                                          self.misalign if layer % 2 else 0, whole=True) for layer in range(self.layers)]
        g, u = self.proj[0][self.gate_i], self.proj[0][self.up_i]
        k0, k1 = g.row0, g.row0 + g.rows
        if g.rows != u.rows or g.rows % 128 or k0 % 64:
            raise ValueError("the K-sharded down projection needs gate/up slices that are multiples of 128 rows")
        rms_src = {"src0": base + off_parts, "src_parts": world, "src_part_stride": part_stride, "sum_out": self.d.data_ptr()}
        stages = []
        for layer in range(self.layers if layers is None else layers):
            jobs, outs = [], []
            for p, o in zip(self.proj[layer], self.outs):
                if p.job is not None:
                    jobs.append(p.job)
                    outs.append(o.data_ptr() + 4 * p.row0)
            first = layer == 0
            head = {"x_kind": capi.X_BF16, "src0": self.x.data_ptr()} if first else {"x_kind": capi.X_RMS, **rms_src}
            stages.append({**head, "k": self.hidden, "eps": 1e-6, "x_bf16_out": 0 if first else self.x.data_ptr(),
                           "jobs": jobs, "outputs": outs})
            mine = off_parts + rank * part_stride
            stages.append({"x_kind": capi.X_SWIGLU, "k": k1 - k0, "k_total": self.inter, "k_begin": k0,
                           "src0": self.outs[self.gate_i].data_ptr() + 4 * k0, "src1": self.outs[self.up_i].data_ptr() + 4 * k0,
                           "x_bf16_out": self.h.data_ptr() + 2 * k0, "jobs": [self.down_whole[layer].job],
                           "outputs": [base + mine],
                           "peer_outputs": [[0 if r == rank else arena[r] + mine for r in range(world)] + [0] * (8 - world)]})
        p = self.lm_head
        self.logits = torch.zeros(max(p.rows, 1), dtype=torch.float32, device=self.device)
        stages.append({"x_kind": capi.X_RMS, **rms_src, "k": self.hidden, "eps": 1e-6,
                       "x_bf16_out": self.x.data_ptr(), "jobs": [p.job], "outputs": [self.logits.data_ptr()]})
        peers = {"world": world, "rank": rank, "flags": [a + off_flags for a in arena], "cand": [a + off_cand for a in arena]}
        if arenas is None:
            dist.barrier()  # every arena is mapped everywhere before the first launch
        return rt.chain_create(stages, self.logits.data_ptr(), p.rows, p.row0, self.token.data_ptr(), self.best.data_ptr(), peers)

    def decode_token(self, stream: int = 0, gather=None, layers=None) -> None:
        """Enqueue one token on `stream` (a raw cudaStream_t). `gather(tensor, proj)` makes a row-sharded
        output whole on every rank; it is None on one GPU. `layers`: only the first so many layers, then lm_head."""
        rt = self.rt
        for layer in range(self.layers if layers is None else layers):
            projs = self.proj[layer]
            self._grouped(self.x.data_ptr(), self.hidden, projs, self.outs, stream)
            gate, up = self.outs[self.gate_i], self.outs[self.up_i]
            if gather is not None:
                gather(gate, projs[self.gate_i])
                gather(up, projs[self.up_i])
            rt.swiglu_device(gate.data_ptr(), up.data_ptr(), self.inter, 0, self.h.data_ptr(), stream)
            self._grouped(self.h.data_ptr(), self.inter, [self.down[layer]], [self.d], stream)
            if gather is not None:
                gather(self.d, self.down[layer])
            rt.rms_unit_bf16_device(self.d.data_ptr(), 1, self.hidden, 1e-6, self.x.data_ptr(), stream)
        p = self.lm_head
        if p.job is not None:
            rt.argmax_batch_device(self.x.data_ptr(), capi.Q4B_BF16, 1, self.hidden, p.job, p.row0,
                                   self.token.data_ptr(), self.best.data_ptr(), stream)
