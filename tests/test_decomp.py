"""The streaming kernel's work split, checked on the CPU: every (tile, chunk) unit belongs to exactly one
warp, the contributor range of a tile is what the ranges imply, partial slots never collide, and a warp
is the first contributor of at most one split tile (that warp's index is the tile's counter)."""
import ctypes as C
import os
import subprocess
import tempfile

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def shim():
    out = os.path.join(tempfile.mkdtemp(prefix="q4decomp"), "shim.so")
    subprocess.check_call(["g++", "-O1", "-shared", "-fPIC", "-o", out, os.path.join(ROOT, "tests", "decomp_shim.cpp")])
    lib = C.CDLL(out)
    lib.shim_begin.restype = C.c_uint64
    lib.shim_begin.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]
    lib.shim_owner.restype = C.c_uint32
    lib.shim_owner.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint64]
    lib.shim_contributors.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
    lib.shim_lane_chunks.restype = C.c_uint32
    lib.shim_slot.restype = C.c_uint32
    lib.shim_slot.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
    lib.shim_rows_part_begin.restype = C.c_uint32
    lib.shim_rows_part_begin.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
    lib.shim_rows_plan.restype = C.c_uint32
    lib.shim_rows_plan.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32)]
    return lib


CONFIGS = [(1, 1, 1), (3, 1, 3), (16, 1, 8), (5, 40, 64), (7, 3, 21), (7, 3, 20), (64, 40, 96), (33, 136, 240), (100, 5, 37), (9, 7, 63), (2, 40, 64)]


@pytest.mark.parametrize("tiles,cpt,workers", CONFIGS)
def test_split_is_a_partition_with_consistent_bookkeeping(shim, tiles, cpt, workers):
    units = tiles * cpt
    assert workers <= units  # the launcher never starts more warps than units, so no warp is idle
    begins = [shim.shim_begin(units, cpt, workers, w) for w in range(workers + 1)]
    assert begins[0] == 0 and begins[-1] == units and all(a <= b for a, b in zip(begins, begins[1:]))
    assert max(b - a for a, b in zip(begins, begins[1:])) - min(b - a for a, b in zip(begins, begins[1:])) <= 1
    owner = [None] * units
    for w in range(workers):
        for u in range(begins[w], begins[w + 1]):
            assert owner[u] is None
            owner[u] = w
    assert all(o is not None for o in owner)
    for u in range(units):
        assert shim.shim_owner(units, cpt, workers, u) == owner[u]
    first_of = {}
    for t in range(tiles):
        f, l = C.c_uint32(), C.c_uint32()
        shim.shim_contributors(units, cpt, workers, t, C.byref(f), C.byref(l))
        who = sorted(set(owner[t * cpt:(t + 1) * cpt]))
        assert who == list(range(f.value, l.value + 1))  # contiguous, nobody idle in between
        if len(who) > 1:
            assert f.value not in first_of, "a warp may be the first contributor of one split tile only"
            first_of[f.value] = t
            slots = [shim.shim_slot(units, cpt, workers, w, t) for w in who]
            assert len(set(slots)) == len(slots)
            for w, s in zip(who, slots):
                assert s // 2 == w
            # the kernel's shortcut: only the first contributor can be in its second slot, and only when its range
            # starts before the tile does
            assert slots == [2 * w + (1 if (w == who[0] and begins[w] < t * cpt) else 0) for w in who]
    # a warp touches at most two split tiles (head and tail), and they use different slots
    for w in range(workers):
        mine = sorted({u // cpt for u in range(begins[w], begins[w + 1])})
        split = [t for t in mine if len(set(owner[t * cpt:(t + 1) * cpt])) > 1]
        assert len(split) <= 2
        assert len({shim.shim_slot(units, cpt, workers, w, t) for t in split}) == len(split)


@pytest.mark.parametrize("k", [64, 128, 192, 640, 1024])
@pytest.mark.parametrize("mis", [0, 1, 2, 4, 7, 15])
def test_byte_addressed_variant_never_reads_outside_the_tensors(shim, k, mis):
    """Address arithmetic of the byte-addressed streaming kernel, on the CPU: every aligned 16-byte window it asks for
    holds at least one byte of the weight row it belongs to, and every parameter it loads is a group of that row. A
    caller's tensors (q4b_matvec_noalloc) therefore need no padding: only 16-byte blocks that the tensors themselves
    touch are read, whatever the byte alignment and for odd group counts too."""
    groups, row_bytes = k // 64, k // 2
    cpt = (groups + 1) // 2
    full_chunks = groups // 2
    for rows in (1, 3):
        base = 4096 + mis  # the tensor starts `mis` bytes past a 16-byte boundary
        lo, hi = base, base + rows * row_bytes
        first_block, last_block = lo // 16, (hi - 1) // 16
        for r in range(rows):
            row_lo, row_hi = base + r * row_bytes, base + (r + 1) * row_bytes
            for c in range(cpt):
                has_b = c < full_chunks
                for t in range(4):
                    window = row_lo + c * 64 + t * 16 - mis  # what the kernel computes: aligned by construction
                    assert window % 16 == 0
                    wanted = [window] if shim.shim_window_wanted(t, mis, int(has_b)) else []
                    if t == 3 and shim.shim_fifth_window_wanted(mis, int(has_b)):
                        wanted.append(window + 16)
                    for a in wanted:
                        assert a < row_hi and a + 16 > row_lo, (r, c, t, a)       # holds bytes of this row
                        assert first_block <= a // 16 <= last_block
                    # everything the lane later reads back from shared memory for an existing group was requested
                    if t < 2 or has_b:
                        need = {window} | ({window + 16} if mis else set())
                        got = set()
                        for tt in range(4):
                            w2 = row_lo + c * 64 + tt * 16 - mis
                            if shim.shim_window_wanted(tt, mis, int(has_b)):
                                got.add(w2)
                            if tt == 3 and shim.shim_fifth_window_wanted(mis, int(has_b)):
                                got.add(w2 + 16)
                        assert need <= got, (r, c, t)
            for t in range(4):
                n = shim.shim_lane_chunks(groups, t)
                assert n == len([c for c in range(cpt) if 2 * c + (t >> 1) < groups])


@pytest.mark.parametrize("k", [512, 1024, 5120, 17408, 32768])
@pytest.mark.parametrize("tiles", [1, 13, 320, 1088, 2176, 15520])
@pytest.mark.parametrize("cap", [12, 24])
@pytest.mark.parametrize("tw", [1, 2])
def test_short_batch_k_split(shim, k, tiles, cap, tw):
    """The short-batch kernel's cut of the K range: parts begin at multiples of four chunks, are never empty, never
    longer than what a block can hold, and together cover every chunk exactly once; the chosen split keeps whole
    blocks per part on a 148-SM GPU."""
    cpt = k // 128
    longest = C.c_uint32(0)
    parts = shim.shim_rows_plan(cpt, tiles, 148, cap, tw, C.byref(longest))
    if (cpt // 4 + 31) // 32 * 4 > cap and parts == 0:
        return  # even 32 parts are too long for the block: the caller falls back to the general kernel
    assert 1 <= parts <= 32 and parts <= cpt // 4
    begins = [shim.shim_rows_part_begin(cpt, parts, p) for p in range(parts + 1)]
    assert begins[0] == 0 and begins[-1] == cpt
    sizes = [b - a for a, b in zip(begins, begins[1:])]
    assert all(s > 0 and s % 4 == 0 for s in sizes) and all(b % 4 == 0 for b in begins)
    assert max(sizes) <= longest.value <= cap
    assert 148 // parts >= 1


def test_short_batch_k_split_prefers_one_round(shim):
    """The benchmark's shapes: the down projection (320 tiles, K = 17408) is cut seven ways so that every warp of
    the grid has exactly one tile; gate and up together (2176 tiles, K = 5120) in two parts, two tiles per warp."""
    longest = C.c_uint32(0)
    assert shim.shim_rows_plan(136, 320, 148, 24, 1, C.byref(longest)) == 7 and longest.value == 20
    assert shim.shim_rows_plan(40, 2176, 148, 24, 1, C.byref(longest)) == 2 and longest.value == 20
    # two tiles per warp: gate and up together are one item per warp of a two-part grid
    assert shim.shim_rows_plan(40, 2176, 148, 21, 2, C.byref(longest)) == 2 and longest.value == 20


def test_signed_digits_from_one_addition():
    """The kernels' digit trick: for |x| <= 2^22, the bytes of (x + 0x808080) ^ 0x808080 are the signed 8-bit digits
    d0, d1, d2 with x = d0 + 256 d1 + 65536 d2 (the activation's fixed-point form on the integer tensor-core path)."""
    import numpy as np

    rng = np.random.default_rng(7)
    x = np.concatenate([rng.integers(-(1 << 22), (1 << 22) + 1, size=200_000), np.array([0, 1, -1, 127, 128, -128, -129, 32767, 32768, -32768, -32769, (1 << 22), -(1 << 22)])]).astype(np.int64)
    z = ((x + 0x808080) & 0xFFFFFFFF) ^ 0x808080
    d = [((z >> (8 * i)) & 0xFF).astype(np.uint8).view(np.int8).astype(np.int64) for i in range(3)]
    assert np.array_equal(d[0] + 256 * d[1] + 65536 * d[2], x)
    assert (z >> 24 == 0).all()
    # a group's integer dot product put together the way the short-batch kernel does it: q0 + (q1 << 8) in int32,
    # + 65536 q2 in fp32; q_d = sum over 64 inputs of w * d_d with 0 <= w <= 15
    w = rng.integers(0, 16, size=(2000, 64)).astype(np.int64)
    xs = rng.integers(-(1 << 22), (1 << 22) + 1, size=(2000, 64)).astype(np.int64)
    zs = ((xs + 0x808080) & 0xFFFFFFFF) ^ 0x808080
    q = [(w * ((zs >> (8 * i)) & 0xFF).astype(np.uint8).view(np.int8).astype(np.int64)).sum(axis=1) for i in range(3)]
    assert (np.abs(q[0] + (q[1] << 8)) < (1 << 31)).all() and (np.abs(q[2]) < (1 << 22)).all()
    exact = (w * xs).sum(axis=1)
    assert np.array_equal(q[0] + 256 * q[1] + 65536 * q[2], exact)
    approx = np.float32(q[2]) * np.float32(65536.0) + (q[0] + (q[1] << 8)).astype(np.float32)
    assert np.all(np.abs(approx.astype(np.float64) - exact) <= np.abs(exact) * 2.0 ** -22 + 4.0)
