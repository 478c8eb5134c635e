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
    lib.shim_slot.restype = C.c_uint32
    lib.shim_slot.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
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
