"""CPU tests of the decomposition solver (cn_compute_decompositions): the seven known-answer
cases of the reference's tests/test_compute_decompositions.cpp:128-396, rebuilt as DAG blobs.
The reference compiles that test with a minimum tile of 64 for every rank
(tests/CMakeLists.txt:40-43); the same minimum is passed here."""
import ctypes as C

from charmnumeric_b200 import _lib, wire
from charmnumeric_b200.wire import Region

MIN_TILE = (C.c_int64 * 3)(64, 64, 64)
OP_COPY = -5


def solve(metas, roots, odf=4, num_pes=1):
    """metas: {name: (shape, offset, tile, final)} -> {name: ArrayMeta} after the solver ran."""
    arr = (_lib.ArrayMeta * len(metas))()
    for i, (name, (shape, offset, tile, final)) in enumerate(metas.items()):
        arr[i].name, arr[i].ndims, arr[i].tile, arr[i].decomp_final = name, len(shape), tile, int(final)
        for d, v in enumerate(shape):
            arr[i].shape[d] = v
        for d, v in enumerate(offset):
            arr[i].offset[d] = v
    blob = wire.dag_blob([wire.Node(0, roots, fusible=True)])
    assert _lib.load().cn_compute_decompositions(arr, len(metas), blob, len(blob), odf, num_pes, MIN_TILE) == 0
    return {a.name: a for a in arr}


def leaf(name, shape):
    return wire.leaf(name, shape)


def test_shifted_copy_uses_absolute_offset():
    A, B = 1, 2
    copy = wire.Ast(B, OP_COPY, shape=(200,), operands=[(leaf(A, (512,)), Region((150,), (350,)))])
    out = solve({A: ((512,), (0,), 64, True), B: ((200,), (0,), 0, False)}, [copy])
    assert out[B].tile == 64 and out[B].offset[0] == 150 and out[B].offset[0] % out[B].tile == 22
    assert out[B].decomp_final


def test_shifted_copy_from_nonzero_source_offset():
    A, B = 1, 2
    copy = wire.Ast(B, OP_COPY, shape=(100,), operands=[(leaf(A, (512,)), Region((70,), (170,)))])
    out = solve({A: ((512,), (132,), 64, True), B: ((100,), (0,), 0, False)}, [copy])
    assert out[B].tile == 64 and out[B].offset[0] == 202 and out[B].offset[0] % 64 == 10


def test_shifted_expression_temp_uses_absolute_representative():
    A, TMP, SET = 1, 10, 11
    tmp = wire.Ast(TMP, wire.OP_ADD, is_temp=True, shape=(200,),
                   operands=[(leaf(A, (512,)), Region((100,), (300,))), (leaf(A, (512,)), Region((150,), (350,)))])
    store = wire.Ast(SET, wire.OP_SET_REGION, shape=(200,), region=Region((200,), (400,)),
                     operands=[(leaf(A, (512,)), None), (wire.Ref(TMP), None)])
    out = solve({A: ((512,), (0,), 64, True), TMP: ((200,), (0,), 0, False)}, [tmp, store])
    assert out[TMP].tile == 64 and out[TMP].offset[0] == 150 and out[TMP].offset[0] % 64 == 22
    assert out[A].offset[0] == 0


def _jacobi(nd, n):
    U, F, TS, TW, SET = 1, 2, 10, 11, 12
    full = (n,) * nd
    inner = (n - 2,) * nd

    def shifted(axis, delta):
        start = [1] * nd
        start[axis] += delta
        return Region(tuple(start), tuple(s + n - 2 for s in start))
    mid = Region((1,) * nd, (n - 1,) * nd)
    ops = []
    for axis in range(nd):
        ops += [(leaf(U, full), shifted(axis, -1)), (leaf(U, full), shifted(axis, 1))]
    metas = {U: (full, (0,) * nd, 64, True), TS: (inner, (0,) * nd, 64, False), TW: (inner, (0,) * nd, 64, False)}
    if nd < 3:
        ops.append((leaf(F, full), mid))
        metas[F] = (full, (0,) * nd, 64, True)
    stencil = wire.Ast(TS, wire.OP_ADD, is_temp=True, shape=inner, operands=ops)
    weighted = wire.Ast(TW, wire.OP_ADD, is_temp=True, shape=inner, operands=[(leaf(U, full), mid), (wire.Ref(TS), None)])
    store = wire.Ast(SET, wire.OP_SET_REGION, shape=inner, region=mid, operands=[(leaf(U, full), None), (wire.Ref(TW), None)])
    out = solve(metas, [stencil, weighted, store])
    want = [1] * nd + [0] * (3 - nd)
    assert out[TS].tile == 64 and out[TW].tile == 64
    assert list(out[TS].offset) == want and list(out[TW].offset) == want


def test_jacobi1d_temp_offset():
    _jacobi(1, 129)


def test_jacobi2d_temp_offset():
    _jacobi(2, 129)


def test_jacobi3d_temp_offset():
    _jacobi(3, 65)


def test_strided_copy_reduces_tile_and_sets_offset():
    A, B = 1, 2
    copy = wire.Ast(B, OP_COPY, shape=(100,), operands=[(leaf(A, (512,)), Region((2,), (202,), (2,)))])
    out = solve({A: ((512,), (0,), 128, True), B: ((100,), (0,), 128, False)}, [copy])
    assert out[B].tile == 64 and out[B].offset[0] == 1 and out[B].offset[0] % out[B].tile == 1


def test_tiles_without_a_dag_follow_the_minimum_and_the_tile_count_cap():
    arr = (_lib.ArrayMeta * 2)()
    arr[0].name, arr[0].ndims, arr[0].tile = 1, 2, 0
    arr[0].shape[0] = arr[0].shape[1] = 2048
    arr[1].name, arr[1].ndims, arr[1].tile = 2, 1, 100
    arr[1].shape[0] = 1 << 28
    assert _lib.load().cn_compute_decompositions(arr, 2, None, 0, 4, 4, None) == 0
    # 2048^2 on 4 PEs, odf 4: minimum 512 gives 16 tiles, allowed; 2^28 elements: 2^24 per tile
    assert arr[0].tile == 512 and arr[1].tile == 1 << 24
