"""CPU-only tests of the host side: the C ABI library loads and exports every declared
symbol, the wire format round-trips and rejects malformed input, the DAG-group compiler
classifies and compiles groups, the frontend groups ops the way the backend expects, and
the product path refuses to run without a GPU."""
import ctypes as C
import re
import struct
from pathlib import Path

import numpy as np
import pytest

import charmnumeric_b200 as cnp
from charmnumeric_b200 import _lib, frontend as F, wire
from charmnumeric_b200._lib import CnError

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "cnb200.h").read_text()
    declared = set(re.findall(r"\b(cn_[a-z_0-9]+)\s*\(", header))
    assert len(declared) >= 25
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in cnb200.h but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes signature table out of step with the header"
    assert lib.cn_version() >= 100
    assert _lib.status_string(0) == "ok"


def test_no_gpu_means_loud_failure():
    """The product path has no CPU fallback: without a device, context creation fails."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(CnError) as e:
        cnp.Context(device=0)
    assert e.value.status == 15


def test_product_package_never_touches_the_oracle():
    for path in (ROOT / "charmnumeric_b200").rglob("*"):
        if path.suffix in (".py", ".cpp", ".hpp", ".cu", ".cuh") and "_build" not in path.parts:
            text = path.read_text()
            assert not re.search(r"^\s*(from|import)\s+\.*oracle|libcn_oracle|cn_oracle|oracle/", text,
                                 re.M), path


# ---- wire format ------------------------------------------------------------------------------

def _jacobi_node(n=16):
    u = lambda: wire.leaf(1, (n, n))  # noqa: E731
    R = lambda a, b, c, d: wire.Region((a, c), (b, d))  # noqa: E731
    s = (n - 2, n - 2)
    return wire.Node(0, [
        wire.Ast(100, wire.OP_ADD, is_temp=True, shape=s, operands=[(u(), R(0, n - 2, 1, n - 1)), (u(), R(2, n, 1, n - 1))]),
        wire.Ast(101, wire.OP_ADD, is_temp=True, shape=s, operands=[(wire.Ref(100), None), (u(), R(1, n - 1, 0, n - 2))]),
        wire.Ast(102, wire.OP_ADD, is_temp=True, shape=s, operands=[(wire.Ref(101), None), (u(), R(1, n - 1, 2, n))]),
        wire.Ast(103, wire.OP_MUL, is_temp=True, shape=s, operands=[(wire.scalar(0.25), None), (wire.Ref(102), None)]),
        wire.Ast(104, wire.OP_SET_REGION, shape=s, region=R(1, n - 1, 1, n - 1), operands=[(u(), None), (wire.Ref(103), None)]),
    ])


def test_region_encoding_matches_reference_layout():
    """ArrayRegion.serialize: int is_global; [int ndims; (start, stop, step) * ndims], 'i'."""
    assert wire.pack_region(None) == struct.pack("<i", 1)
    r = wire.Region((1, 2), (5, 9), (1, 3))
    assert wire.pack_region(r) == struct.pack("<ii", 0, 2) + struct.pack("<iii", 1, 5, 1) + struct.pack("<iii", 2, 9, 3)
    assert r.shape() == (4, 3)


def test_dag_blob_parses():
    blob = wire.dag_blob([_jacobi_node(), wire.Node(1, [wire.Ast(7, wire.OP_CREATE, shape=(4, 4))], fusible=False)], deletes=[3, 4])
    assert cnp.dag_check(blob) == (2, 6)


@pytest.mark.parametrize("mutate", ["magic", "truncate", "trailing", "rank", "step"])
def test_malformed_blobs_are_rejected(mutate):
    blob = bytearray(wire.dag_blob([_jacobi_node()]))
    if mutate == "magic":
        blob[0:4] = b"XXXX"
    elif mutate == "truncate":
        blob = blob[:len(blob) // 2]
    elif mutate == "trailing":
        blob += b"\0\0\0\0"
    elif mutate == "rank":
        node = wire.Node(0, [wire.Ast(1, wire.OP_CREATE, shape=(2, 2, 2, 2))], fusible=False)
        blob = bytearray(wire.dag_blob([node]))
    elif mutate == "step":
        node = _jacobi_node()
        node.roots[0].operands[0] = (node.roots[0].operands[0][0], wire.Region((0, 1), (14, 15), (0, 1)))
        blob = bytearray(wire.dag_blob([node]))
    with pytest.raises(CnError) as e:
        cnp.dag_check(bytes(blob))
    assert e.value.status == 2


# ---- DAG-group compiler -------------------------------------------------------------------------

def test_jacobi_group_lowers_to_vectorised_copy_through_kernel():
    src, nbytes = cnp.group_compile_check(_jacobi_node(64))
    assert nbytes > 0
    assert "double2" in src                      # 128-bit loads/stores
    assert "old0" in src and "act0" in src       # out-of-place sweep with copy-through
    assert "__restrict__" in src
    assert src.count("cn_exp") == 0


def test_odd_width_falls_back_to_scalar_loads():
    src, _ = cnp.group_compile_check(_jacobi_node(17))
    assert "typedef double2" not in src


def test_group_with_fused_sum_has_deterministic_finish():
    n = 256
    a, b = wire.leaf(1, (n,)), wire.leaf(2, (n,))
    node = wire.Node(0, [
        wire.Ast(10, wire.OP_MUL, is_temp=True, shape=(n,), operands=[(a, None), (b, None)]),
        wire.Ast(11, wire.OP_SUM, shape=(1,), operands=[(wire.Ref(10), None)]),
    ])
    src, _ = cnp.group_compile_check(node)
    assert "cn_grid_ticket" in src and "cn_sum_partials" in src


def test_strided_group_compiles():
    n = 17
    fine, coarse = wire.leaf(1, (n, n)), wire.leaf(2, (9, 9))
    node = wire.Node(0, [wire.Ast(5, wire.OP_SET_REGION, shape=(7, 7), region=wire.Region((1, 1), (8, 8)),
                                  operands=[(coarse, None), (fine, wire.Region((2, 2), (15, 15), (2, 2)))])])
    src, _ = cnp.group_compile_check(node)
    assert "in_str" in src


@pytest.mark.parametrize("case,status", [("opcode", 6), ("shape", 4), ("hazard", 11), ("exp_int", 7)])
def test_lowering_errors(case, status):
    n = 8
    a, b = wire.leaf(1, (n,)), wire.leaf(2, (n + 1,))
    if case == "opcode":
        node = wire.Node(0, [wire.Ast(10, wire.OP_MATMATMUL, shape=(n,), operands=[(a, None), (a, None)])])
    elif case == "shape":
        node = wire.Node(0, [wire.Ast(10, wire.OP_ADD, shape=(n,), operands=[(a, None), (b, None)])])
    elif case == "hazard":
        node = wire.Node(0, [
            wire.Ast(10, wire.OP_SET_REGION, shape=(n - 1,), region=wire.Region((0,), (n - 1,)),
                     operands=[(a, None), (a, wire.Region((1,), (n,)))]),
            wire.Ast(11, wire.OP_ADD, shape=(n - 2,), operands=[(a, wire.Region((2,), (n,))), (a, wire.Region((0,), (n - 2,)))]),
        ])
    else:
        ai = wire.leaf(1, (n,), dtype=wire.I32)
        node = wire.Node(0, [wire.Ast(10, wire.OP_EXP, shape=(n,), dtype=wire.I32, operands=[(ai, None)])])
    with pytest.raises(CnError) as e:
        cnp.group_compile_check(node)
    assert e.value.status == status


# ---- slab partition -------------------------------------------------------------------------------

@pytest.mark.parametrize("n0,nranks", [(2048, 1), (2048, 8), (10, 4), (3, 8), (8194, 8), (0, 2)])
def test_partition_covers_rows_exactly_once(n0, nranks):
    lib = _lib.load()
    covered = []
    for r in range(nranks):
        b, e = C.c_int64(), C.c_int64()
        assert lib.cn_partition(n0, nranks, r, C.byref(b), C.byref(e)) == 0
        assert 0 <= b.value <= e.value <= n0
        covered.extend(range(b.value, e.value))
    assert covered == list(range(n0))
    assert lib.cn_partition(n0, nranks, nranks, C.byref(b), C.byref(e)) == 1


# ---- frontend -------------------------------------------------------------------------------------

def test_jacobi_statement_becomes_one_group_with_temporaries():
    u = cnp.zeros((8, 8))
    u[1:-1, 1:-1] = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:])
    items = F.build_nodes(F._state.pending)
    nodes = [n for _, n in items]
    assert [n.fusible for n in nodes] == [False, True]
    roots = nodes[1].roots
    # t1, t2, t3 = ADD (temps), t4 = MUL(0.25, t3) (temp), SET_REGION: the reference's root list
    assert [r.opcode for r in roots] == [0, 0, 0, 2, -4]
    assert [r.is_temp for r in roots[:4]] == [True] * 4
    assert roots[3].operands[0][0].is_scalar and roots[3].operands[0][0].scalar == 0.25
    assert roots[4].region == wire.Region((1, 1), (7, 7))


def test_negation_is_multiplication_by_minus_one():
    a = cnp.ones((4,))
    b = -a
    op = F._state.pending[-1]
    assert op.opcode == 2 and op.operands[1] == -1
    del b


def test_dot_and_matvec_are_their_own_nodes():
    A = cnp.ones((4, 4))
    x = cnp.ones((4,))
    y = A @ x
    s = y @ y
    z = y / s
    nodes = [n for _, n in F.build_nodes(F._state.pending)]
    kinds = [(n.fusible, [r.opcode for r in n.roots]) for n in nodes]
    assert (False, [4]) in kinds and (False, [8]) in kinds
    assert kinds[-1] == (True, [3])
    del z


def test_live_results_are_materialised_dead_ones_are_not():
    a = cnp.ones((4,))
    keep = a + 1.0
    out = (a + 2.0) * keep
    nodes = [n for _, n in F.build_nodes(F._state.pending)]
    roots = nodes[-1].roots
    by_name = {r.result_name: r for r in roots}
    assert not by_name[keep.name].is_temp
    assert not by_name[out.name].is_temp
    assert sum(1 for r in roots if r.is_temp) == 1


def test_index_errors_match_numpy_style():
    a = cnp.zeros((4, 4))
    with pytest.raises(IndexError):
        a[5, 0]
    with pytest.raises(IndexError):
        a[0, 0, 0]
    with pytest.raises(NotImplementedError):
        a[::-1]
    with pytest.raises(ValueError):
        a[::0]
    with pytest.raises(TypeError):
        cnp.zeros((4,), dtype=np.complex64)
    with pytest.raises(ValueError):
        bool(a)
    v = a[1:3][:, 1:4:2]
    assert v.shape == (2, 2) and v._region == wire.Region((1, 1), (3, 4), (1, 2))


def test_shape_mismatch_is_reported_by_the_frontend():
    with pytest.raises(ValueError):
        cnp.zeros((4,)) + cnp.zeros((5,))
    with pytest.raises(ValueError):
        cnp.zeros((4, 3)) @ cnp.zeros((4,))


def test_exp_tables_of_oracle_and_device_are_identical():
    """The oracle's C table and the device table come from two generator scripts; exp and tanh
    are only bit-identical between the two while every entry and the ln2 split agree."""
    import re
    root = Path(__file__).resolve().parent.parent
    dev = (root / "charmnumeric_b200" / "csrc" / "cn_exp_table.inc").read_text()
    orc = (root / "oracle" / "cn_oracle_exp_table.h").read_text()
    hexf = r"-?0x[0-9a-f.]+p[-+]?\d+"

    def block(text, start, end):
        i = text.index(start)
        j = text.index(end, i)
        return [float.fromhex(v) for v in re.findall(hexf, text[i + len(start):j])]
    dev_hi = block(dev, "#define CN_EXP_TABLE_HI", "#define CN_EXP_TABLE_LO")
    dev_lo = block(dev, "#define CN_EXP_TABLE_LO", "#define CN_EXP_TABLE_PAIRS")
    dev_pairs = block(dev, "#define CN_EXP_TABLE_PAIRS", "#define CN_LN2_64_HI")
    orc_hi = block(orc, "CNO_T_HI[64] = {", "};")
    orc_lo = block(orc, "CNO_T_LO[64] = {", "};")
    assert len(dev_hi) == len(dev_lo) == 64 and len(dev_pairs) == 128
    assert [v.hex() for v in dev_hi] == [v.hex() for v in orc_hi]
    assert [v.hex() for v in dev_lo] == [v.hex() for v in orc_lo]
    assert [v.hex() for v in dev_pairs[0::2]] == [v.hex() for v in orc_hi]
    assert [v.hex() for v in dev_pairs[1::2]] == [v.hex() for v in orc_lo]
    consts_dev = [float.fromhex(re.search(name + r"\s+(" + hexf + ")", dev).group(1))
                  for name in ("CN_LN2_64_HI", "CN_LN2_64_LO", "CN_INV_LN2_64")]
    consts_orc = [float.fromhex(re.search(name + r"\s*=\s*(" + hexf + ")", orc).group(1))
                  for name in ("CNO_C_HI", "CNO_C_LO", "CNO_INV")]
    assert [v.hex() for v in consts_dev] == [v.hex() for v in consts_orc]


def _pending_nodes():
    return [n for kind, n in F.build_nodes(F._state.pending) if kind == "node"]


def test_direction_update_and_stencil_compile_as_one_kernel():
    """Host side of the producer inlining: `p = r + beta p` and the 5-point stencil over p
    become one kernel that reads r and p and writes p and Ap."""
    from charmnumeric_b200.context import fuse_check
    cnp.reset_frontend_state()
    m = 66
    p, r, Ap, beta = cnp.zeros((m, m)), cnp.zeros((m, m)), cnp.zeros((m, m)), cnp.zeros((1,))
    F._state.pending = []
    p[...] = r + beta * p
    Ap[1:-1, 1:-1] = 4.0 * p[1:-1, 1:-1] - p[:-2, 1:-1] - p[2:, 1:-1] - p[1:-1, :-2] - p[1:-1, 2:]
    nodes = _pending_nodes()
    assert len(nodes) == 2
    src = fuse_check(nodes[0], nodes[1])
    # the staged form: the stencil reads a stand-in whose tiles the kernel computes from r and p
    assert src is not None and "cn_group_shifted2d_i1o2" in src and "Pin1" in src and "ring" in src
    import os
    os.environ["CN_FUSE_PRODUCERS"] = "1"
    try:
        cloned = fuse_check(nodes[0], nodes[1])  # the form that recomputes at every stencil point
    finally:
        del os.environ["CN_FUSE_PRODUCERS"]
    assert cloned is not None and "cn_group_shifted2d_i2o2" in cloned
    # a stencil that assigns into the producer's own input must not fuse
    cnp.reset_frontend_state()
    F._state.pending = []
    p2, r2, beta2 = cnp.zeros((m, m)), cnp.zeros((m, m)), cnp.zeros((1,))
    F._state.pending = []
    p2[...] = r2 + beta2 * p2
    r2[1:-1, 1:-1] = 0.25 * (p2[:-2, 1:-1] + p2[2:, 1:-1] + p2[1:-1, :-2] + p2[1:-1, 2:])
    nodes = _pending_nodes()
    assert len(nodes) == 2 and fuse_check(nodes[0], nodes[1]) is None
    # and neither does a pair whose first node is not a whole-array assignment
    cnp.reset_frontend_state()
    F._state.pending = []
    p3, r3 = cnp.zeros((m, m)), cnp.zeros((m, m))
    F._state.pending = []
    p3[1:-1, :] = r3[1:-1, :] + 1.0
    r3[1:-1, 1:-1] = p3[:-2, 1:-1] + p3[2:, 1:-1]
    nodes = _pending_nodes()
    assert fuse_check(nodes[0], nodes[-1]) is None
    cnp.reset_frontend_state()


def test_scalar_node_behind_a_fused_reduction_compiles_into_its_kernel():
    """Host side of the scalar tail: CG's x, r update with its fused r.r, followed by
    beta = r.r / rtr and rtr = r.r on size-1 arrays, is one kernel whose finishing thread
    evaluates the size-1 arithmetic."""
    from charmnumeric_b200.context import tail_check
    from charmnumeric_b200 import wire
    cnp.reset_frontend_state()
    m = 66
    x, r, p, Ap = (cnp.zeros((m, m)) for _ in range(4))
    alpha, beta, rtr = cnp.zeros((1,)), cnp.zeros((1,)), cnp.zeros((1,))
    F._state.pending = []
    x[...] = x + alpha * p
    r[...] = r - alpha * Ap
    rr = cnp.dot2d(r, r)
    beta[...] = rr / rtr
    rtr[...] = rr
    nodes = _pending_nodes()
    assert len(nodes) == 3, [len(n.roots) for n in nodes]
    src = tail_check(wire.dag_blob(nodes))
    assert src is not None
    tail = src[src.index("cn_sum_partials"):]
    # operands of the tail sit behind the group's own size-1 operand (alpha): r.r and rtr
    assert "Sb0" in tail and "Sb1" in tail and "a.sout[0]" in tail and "a.sout[1]" in tail
    assert tail.index("a.red[0]") < tail.index("Sb0")     # results are stored before they are read back
    # a last node that is not size-1 arithmetic is no tail
    cnp.reset_frontend_state()
    F._state.pending = []
    x2, r2 = cnp.zeros((m, m)), cnp.zeros((m, m))
    F._state.pending = []
    r2[...] = r2 - 0.5 * x2
    rr2 = cnp.dot2d(r2, r2)
    x2[...] = x2 + rr2 * r2
    nodes = _pending_nodes()
    assert len(nodes) == 3 and tail_check(wire.dag_blob(nodes)) is None
    cnp.reset_frontend_state()
