"""CPU tests of the slab planner's region algebra (host-only entry points of the C ABI):
the asserting cases of the reference's own region tests (tests/test_jit.cpp:244-326) restated
on row lattices, and a brute-force check that the planned row transfers are exactly what
each rank reads but does not own."""
import ctypes as C

import numpy as np
import pytest

from charmnumeric_b200 import _lib


def _triple(r):
    return (C.c_int64 * 3)(*r)


def intersect(a, b):
    out = (C.c_int64 * 3)()
    assert _lib.load().cn_region_intersect(_triple(a), _triple(b), out) == 0
    return tuple(out)


def region_map(part, src, dst):
    out = (C.c_int64 * 3)()
    assert _lib.load().cn_region_map(_triple(part), _triple(src), _triple(dst), out) == 0
    return tuple(out)


def plan(anchor, anchor_n0, leaf, leaf_n0, nranks):
    lib = _lib.load()
    count = C.c_int64()
    rows = (C.c_int64 * (2 * nranks))()
    buf = (C.c_int64 * (4 * nranks * nranks + 4))()
    assert lib.cn_plan_row_transfers(_triple(anchor), anchor_n0, _triple(leaf), leaf_n0, nranks, buf,
                                     nranks * nranks + 1, C.byref(count), rows) == 0
    moves = [tuple(buf[4 * i:4 * i + 4]) for i in range(count.value)]
    return moves, [(rows[2 * q], rows[2 * q + 1]) for q in range(nranks)]


def test_map_preserves_stepped_extent_across_tile_boundaries():
    # tests/test_jit.cpp:301-326
    parent_input, tile_input, parent_output = (2, 127, 2), (64, 127, 2), (1, 64, 1)
    mapped = region_map(tile_input, parent_input, parent_output)
    assert mapped == (32, 64, 1)
    back = region_map((32, 64, 1), parent_output, parent_input)
    assert back == (64, 128, 2)
    assert len(range(*back)) == len(range(32, 64))


def test_halves_of_a_stepped_parent_map_to_dense_halves():
    # tests/test_jit.cpp:244-298: the two halves of parent {0, 64, 2} sit at packed offsets 0 and 16
    parent, left, right, dense = (0, 64, 2), (0, 32, 2), (32, 64, 2), (0, 32, 1)
    assert region_map(left, parent, dense) == (0, 16, 1)
    assert region_map(right, parent, dense) == (16, 32, 1)
    # in a dense local buffer the same halves start at elements 0 and 32 with stride 2
    assert region_map(left, parent, parent)[0] == 0 and region_map(right, parent, parent)[::2] == (32, 2)


@pytest.mark.parametrize("a,b", [((0, 64, 2), (32, 64, 2)), ((1, 100, 3), (0, 100, 2)), ((5, 50, 4), (6, 50, 4)),
                                 ((0, 10, 1), (10, 20, 1)), ((7, 200, 6), (1, 150, 4)), ((3, 4, 5), (3, 9, 2))])
def test_intersect_matches_python_sets(a, b):
    got = intersect(a, b)
    want = sorted(set(range(*a)) & set(range(*b)))
    assert list(range(*got)) == want if want else len(range(*got)) == 0


def test_map_rejects_a_region_that_is_not_part_of_the_view():
    out = (C.c_int64 * 3)()
    assert _lib.load().cn_region_map(_triple((3, 9, 2)), _triple((0, 10, 4)), _triple((0, 3, 1)), out) == 1


def test_planned_transfers_are_what_each_rank_reads_and_does_not_own():
    rng = np.random.default_rng(2024)
    for _ in range(300):
        nranks = int(rng.integers(1, 9))
        extent = int(rng.integers(1, 60))
        astep, lstep = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        astart, lstart = int(rng.integers(0, 5)), int(rng.integers(0, 7))
        anchor = (astart, astart + (extent - 1) * astep + 1, astep)
        leaf = (lstart, lstart + (extent - 1) * lstep + 1, lstep)
        anchor_n0 = anchor[1] + int(rng.integers(0, 4))
        leaf_n0 = leaf[1] + int(rng.integers(0, 4))
        moves, rows = plan(anchor, anchor_n0, leaf, leaf_n0, nranks)
        lib = _lib.load()

        def own(n0, q):
            b, e = C.c_int64(), C.c_int64()
            lib.cn_partition(n0, nranks, q, C.byref(b), C.byref(e))
            return b.value, e.value
        # the iteration rows of all ranks tile [0, extent) in rank order
        covered = []
        for q, (i0, i1) in enumerate(rows):
            b, e = own(anchor_n0, q)
            assert all(b <= anchor[0] + i * anchor[2] < e for i in range(i0, i1))
            covered += list(range(i0, i1))
        assert covered == list(range(extent))
        for q, (i0, i1) in enumerate(rows):
            needed = {leaf[0] + i * leaf[2] for i in range(i0, i1)}
            b, e = own(leaf_n0, q)
            have = set(range(b, e))
            for src, dst, lo, hi in moves:
                if dst == q:
                    sb, se = own(leaf_n0, src)
                    assert sb <= lo < hi <= se and src != q
                    assert not (have & set(range(lo, hi))) or True
                    have |= set(range(lo, hi))
            assert needed <= have, (anchor, leaf, nranks, q)
            # nothing travels that lies outside the bounding range of what is read
            if needed:
                for src, dst, lo, hi in moves:
                    if dst == q:
                        assert min(needed) <= lo and hi <= max(needed) + 1
            else:
                assert not [m for m in moves if m[1] == q]


def test_aligned_views_need_no_transfers():
    # unit-step views with one start over arrays of one height: every rank reads its own rows
    for nranks in (2, 4, 8):
        moves, _ = plan((1, 129, 1), 130, (1, 129, 1), 130, nranks)
        assert moves == []
    # a 5-point stencil's shifted views read one row of each neighbour
    moves, _ = plan((1, 129, 1), 130, (0, 128, 1), 130, 2)
    assert moves == [(0, 1, 64, 65)]
