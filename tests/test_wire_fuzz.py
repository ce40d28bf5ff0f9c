"""The DAG blob reader against damaged input (host only, no GPU): truncation at every length,
flipped bytes, and counts that claim far more than the bytes could hold must all come back as
a status code -- never a crash, a hang or a large allocation.  The reference trusts its DAG
bytes (DAG::deserialize, src/dag_group_receive.cpp:192); this reader sits on the same boundary."""
import ctypes as C
import struct

import numpy as np
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

import charmnumeric_b200 as cnp
from charmnumeric_b200 import _lib, wire
from charmnumeric_b200 import frontend as F


def _valid_blob():
    cnp.reset_frontend_state()
    u = cnp.zeros((34, 40))
    u[0, :] = 1.0
    for _ in range(2):
        new = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:])
        d = new - u[1:-1, 1:-1]
        u[1:-1, 1:-1] = new
        s = cnp.sum(d * d)
    y = cnp.ones((34, 40)) @ cnp.ones((40,))
    items = F.build_nodes(F._state.pending)
    cnp.reset_frontend_state()
    nodes = [n for kind, n in items if kind == "node"]
    return wire.dag_blob(nodes, deletes=[3, 4])


BLOB = _valid_blob()
LIB = _lib.load()


def _check(blob):
    err = C.create_string_buffer(512)
    n_nodes, n_roots = C.c_int(0), C.c_int(0)
    return LIB.cn_dag_check(bytes(blob), len(blob), C.byref(n_nodes), C.byref(n_roots), err, len(err)), n_nodes.value


def test_the_undamaged_blob_parses():
    rc, n = _check(BLOB)
    assert rc == 0 and n >= 3


def test_every_truncation_is_rejected():
    for cut in range(len(BLOB)):
        rc, _ = _check(BLOB[:cut])
        assert rc == 2, cut            # CN_STATUS_BAD_BLOB
    rc, _ = _check(BLOB + b"\0")
    assert rc == 2                     # trailing bytes


@pytest.mark.parametrize("offset", [8, 12 + 16, 12 + 20])   # n_nodes, n_deps and n_roots of node 0
@pytest.mark.parametrize("value", [-1, 1 << 20, 1 << 22, 0x7fffffff])
def test_counts_beyond_the_remaining_bytes_are_rejected(offset, value):
    damaged = bytearray(BLOB)
    damaged[offset:offset + 4] = struct.pack("<i", value)
    rc, _ = _check(damaged)
    assert rc == 2


@settings(max_examples=300, deadline=None)
@given(st.lists(st.tuples(st.integers(0, len(BLOB) - 1), st.integers(0, 255)), min_size=1, max_size=8))
def test_flipped_bytes_never_crash(edits):
    damaged = bytearray(BLOB)
    for pos, val in edits:
        damaged[pos] = val
    rc, _ = _check(damaged)
    assert rc in (0, 2)


@settings(max_examples=200, deadline=None)
@given(st.binary(min_size=0, max_size=256))
def test_arbitrary_bytes_never_crash(data):
    rc, _ = _check(b"CNB1" + data)
    assert rc in (0, 2)
    assert _check(data)[0] in (0, 2)


def test_group_compile_check_rejects_damaged_nodes():
    """The single-group entry point (cn_group_compile_check) reads the same grammar."""
    src = C.create_string_buffer(1 << 16)
    err = C.create_string_buffer(1024)
    nb = C.c_int64(0)
    node = BLOB[12:12 + 200]           # a prefix of node 0: truncated group blob
    rc = LIB.cn_group_compile_check(node, len(node), src, len(src), C.byref(nb), err, len(err))
    assert rc == 2
    assert np.frombuffer(err.raw[:8], dtype=np.uint8).any()   # a message came back


def _fusible_group_blobs():
    cnp.reset_frontend_state()
    u = cnp.zeros((34, 40))
    u[0, :] = 1.0
    new = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:])
    d = new - u[1:-1, 1:-1]
    u[1:-1, 1:-1] = new
    s = cnp.sum(d * d)
    coarse, fine = cnp.zeros((9, 9)), cnp.ones((17, 17))
    coarse[1:-1, 1:-1] = fine[2:-2:2, 2:-2:2]
    a = cnp.ones((100,))
    b = cnp.exp(a) / (1 + cnp.abs(a))
    items = F.build_nodes(F._state.pending)
    cnp.reset_frontend_state()
    return [n.pack() for kind, n in items if kind == "node" and n.fusible]


def test_damaged_groups_never_crash_the_compiler():
    """Well-formed but wrong groups (bad opcodes, ranks, regions, operand references, extents)
    must be turned away by the lowering with a status: 150 seeded mutations of real groups go
    through parse -> lower -> generate -> NVRTC, and every one comes back with a status code
    (ok, bad blob, shape mismatch, bad dtype, bad opcode, unsupported, hazard or limit)."""
    import random
    rng = random.Random(20260)
    groups = _fusible_group_blobs()
    assert len(groups) >= 4
    src = C.create_string_buffer(1 << 17)
    err = C.create_string_buffer(2048)
    nb = C.c_int64(0)
    seen = set()
    for _ in range(150):
        g = bytearray(rng.choice(groups))
        for _ in range(rng.randint(1, 3)):
            pos = rng.randrange(len(g))
            if rng.random() < 0.5:
                g[pos] = rng.randrange(256)
            else:
                pos -= pos % 4
                g[pos:pos + 4] = struct.pack("<i", rng.choice([-1, 0, 1, 2, 3, 7, 2 ** 31 - 1, -2 ** 31, 10 ** 6,
                                                               rng.randrange(-5, 50)]))
        rc = LIB.cn_group_compile_check(bytes(g), len(g), src, len(src), C.byref(nb), err, len(err))
        seen.add(rc)
        assert rc in (0, 2, 4, 5, 6, 7, 11, 13), (rc, err.value)
    assert 0 in seen and 2 in seen
