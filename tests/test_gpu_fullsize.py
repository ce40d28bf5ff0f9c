"""GPU tests at the configured (full) sizes, and cross-checks between kernel variants.

Full-size fields are too large to pull back element by element in a test run, so the checks at
those sizes go through scalars the oracle can produce from the same seeded inputs (residuals,
dot products, checksums) and through properties that do not depend on size (the TMA-staged and
the cache-served stencil kernels must agree bit for bit; fused and unfused reductions must
agree to the reduction tolerance; matvec is linear).
"""
import ctypes as C

import numpy as np
import pytest

import charmnumeric_b200 as cnp
from charmnumeric_b200 import frontend as F
from tests import test_gpu_parity as G
from tests.helpers import assert_bit_exact, assert_rel, run_both

pytestmark = pytest.mark.gpu
RTOL = 1e-10


def _run_gpu_only(interface, prog):
    cnp.reset_frontend_state()
    outs = prog()
    F.execute(interface)
    return {k: interface.context.get(v.name).reshape(v.shape) for k, v in outs.items()}


@pytest.mark.parametrize("prog", [
    G._jacobi2d_program(514, 1030, 6, res_every=3),
    G._jacobi3d_program((70, 52, 260), 4),
    G._cg_poisson_program(322, 6),
], ids=["jacobi2d", "jacobi3d", "cg"])
def test_staged_and_cache_served_kernels_agree_bit_for_bit(interface, prog):
    ctx = interface.context
    results = []
    try:
        for level in (0, 2):
            ctx.set_option("staged", level)
            results.append(_run_gpu_only(interface, prog))
    finally:
        ctx.set_option("staged", 1)
    a, b = results
    # CG iterates depend on the dot products, whose summation order differs between the two
    # kernels; the Jacobi fields must match bit for bit
    exact = "rtr0" not in a
    for k in a:
        if a[k].size > 1 and exact:
            assert a[k].tobytes() == b[k].tobytes(), k
        else:
            scale = np.max(np.abs(b[k]))
            assert np.max(np.abs(a[k] - b[k])) <= RTOL * scale, k


def test_fused_and_unfused_reductions_agree(interface):
    ctx = interface.context
    results = []
    try:
        for fuse in (1, 0):
            ctx.set_option("fuse_reductions", fuse)
            before = ctx.stats()["fused_reductions"]
            results.append(_run_gpu_only(interface, G._cg_poisson_program(130, 10)))
            fused = ctx.stats()["fused_reductions"] - before
            assert (fused > 0) == bool(fuse)
    finally:
        ctx.set_option("fuse_reductions", 1)
    assert_rel(results[0], results[1], RTOL)


def test_config2_chain_sum_full_size(interface, oracle_mod):
    """C2: n = 2^28, s = sum(exp(-a*a)*b + sqrt(|a|) - 0.5*b*b + a/(1+|b|))."""
    n = 1 << 28

    def prog():
        a = cnp.random.uniform((n,), seed=0x5EED + 2, low=-1.0, high=1.0)
        b = cnp.random.uniform((n,), seed=0x5EED + 22, low=-1.0, high=1.0)
        return {"s": cnp.sum(G._chain(a, b))}
    got = _run_gpu_only(interface, prog)["s"][0]
    a = oracle_mod.randu((n,), 0x5EED + 2, -1.0, 1.0)
    b = oracle_mod.randu((n,), 0x5EED + 22, -1.0, 1.0)
    want = oracle_mod.clib().cno_chain_sum(oracle_mod._ptr(a), oracle_mod._ptr(b), n, 1 << 24)
    assert abs(got - want) <= RTOL * abs(want)


def test_config3_cg_full_size(interface, oracle_mod):
    """C3: 8192 x 8192 unknowns; the r.r history of the first iterations against the oracle."""
    m, iters = 8194, 6
    got = _run_gpu_only(interface, G._cg_poisson_program(m, iters))
    b = np.zeros((m, m))
    b[1:-1, 1:-1] = oracle_mod.randu((m, m), 0x5EED + 3)[1:-1, 1:-1]
    x, r, p, Ap = (np.empty((m, m)) for _ in range(4))
    hist = np.zeros(iters)
    oracle_mod.clib().cno_cg_poisson(oracle_mod._ptr(b), oracle_mod._ptr(x), oracle_mod._ptr(r),
                                     oracle_mod._ptr(p), oracle_mod._ptr(Ap), m, iters,
                                     oracle_mod._ptr(hist), 1 << 22)
    for k in range(iters):
        assert abs(got[f"rtr{k}"][0] - hist[k]) <= RTOL * hist[k], k
    scale = np.max(np.abs(x))
    assert np.max(np.abs(got["x"] - x)) <= RTOL * scale


def test_config5_jacobi3d_full_size(interface, oracle_mod):
    """C5: 1024^3; residual of the second sweep and a checksum of the field."""
    n = 1024

    def prog():
        u = cnp.random.uniform((n, n, n), seed=0x5EED + 5)
        u[0, :, :] = 1.0
        u[-1, :, :] = 0.0
        u[:, 0, :] = 0.0
        u[:, -1, :] = 0.0
        u[:, :, 0] = 0.0
        u[:, :, -1] = 0.0
        c = 1.0 / 6.0
        out = {}
        for it in range(2):
            new = c * (u[:-2, 1:-1, 1:-1] + u[2:, 1:-1, 1:-1] + u[1:-1, :-2, 1:-1]
                       + u[1:-1, 2:, 1:-1] + u[1:-1, 1:-1, :-2] + u[1:-1, 1:-1, 2:])
            d = new - u[1:-1, 1:-1, 1:-1]
            sq = d * d
            u[1:-1, 1:-1, 1:-1] = new
            out[f"res{it}"] = cnp.sum(sq)
            del new, d, sq
        out["checksum"] = cnp.sum(u)
        out["plane"] = u[511, :, :].copy()
        return out
    got = _run_gpu_only(interface, prog)
    u = oracle_mod.randu((n, n, n), 0x5EED + 5)
    u[0] = 1.0
    u[-1] = 0.0
    u[:, 0] = 0.0
    u[:, -1] = 0.0
    u[:, :, 0] = 0.0
    u[:, :, -1] = 0.0
    scratch = np.zeros_like(u)
    res = np.zeros(2)
    oracle_mod.clib().cno_jacobi3d(oracle_mod._ptr(u), oracle_mod._ptr(scratch), n, n, n, 1.0 / 6.0, 2, 1,
                                   oracle_mod._ptr(res), 64)
    for it in range(2):
        assert abs(got[f"res{it}"][0] - res[it]) <= RTOL * res[it]
    want_sum = oracle_mod.dot(u, np.ones(u.size), tile=1 << 24)
    assert abs(got["checksum"][0] - want_sum) <= RTOL * abs(want_sum)
    assert got["plane"].tobytes() == u[511].tobytes()      # one full plane, bit for bit


def test_config4_matvec_properties(interface, oracle_mod):
    """C4: against the oracle at 16384^2 (a matrix the host can hold) and linearity at 65536^2."""
    n = 16384

    def small():
        A = cnp.random.uniform((n, n), seed=0x5EED + 4, low=-1.0 / 256, high=1.0 / 256)
        x = cnp.random.uniform((n,), seed=0x5EED + 44, low=-1.0, high=1.0)
        return {"y": A @ x}
    got = _run_gpu_only(interface, small)["y"]
    A = oracle_mod.randu((n, n), 0x5EED + 4, -1.0 / 256, 1.0 / 256)
    x = oracle_mod.randu((n,), 0x5EED + 44, -1.0, 1.0)
    want = oracle_mod.gemv(A, x, tile=4096)
    assert np.max(np.abs(got - want)) <= RTOL * np.max(np.abs(want))
    del A

    N = 65536

    def full():
        A = cnp.random.uniform((N, N), seed=0x5EED + 4, low=-1.0 / 256, high=1.0 / 256)
        x = cnp.random.uniform((N,), seed=1, low=-1.0, high=1.0)
        y = cnp.random.uniform((N,), seed=2, low=-1.0, high=1.0)
        return {"Ax": A @ x, "Ay": A @ y, "Axy": A @ (x + y)}
    r = _run_gpu_only(interface, full)
    scale = np.max(np.abs(r["Axy"]))
    assert np.max(np.abs(r["Axy"] - (r["Ax"] + r["Ay"]))) <= 1e-12 * scale * 10
    # closed form at the configured size: 256 rows of the seeded matrix are regenerated on the
    # host (element (i, j) is value number i * N + j of the seeded generator) and multiplied by
    # the regenerated x; a kernel that dropped or misplaced columns would not survive this
    xh = oracle_mod.randu((N,), 1, -1.0, 1.0)
    rows = np.unique(np.concatenate([[0, 1, N - 2, N - 1, N // 2 - 1, N // 2],
                                     np.random.default_rng(5).integers(0, N, 250)]))
    worst = 0.0
    for i in rows:
        a_row = oracle_mod.randu((N,), 0x5EED + 4, -1.0 / 256, 1.0 / 256, offset=int(i) * N)
        want_i = oracle_mod.dot(a_row, xh, tile=4096)
        worst = max(worst, abs(r["Ax"][i] - want_i))
    assert worst <= RTOL * np.max(np.abs(r["Ax"])), worst


def test_kernel_abi_compile_and_launch(interface):
    """cn_compile_group / cn_launch_group: the raw kernel ABI with strided views, on memory the
    caller owns (torch tensors here), as the reference's dispatch_kernel is used."""
    import torch
    from charmnumeric_b200 import _lib, wire
    ctx = interface.context
    n0, n1 = 37, 50
    a_leaf, b_leaf = wire.leaf(1, (n0, n1)), wire.leaf(2, (n0, n1))
    ra = wire.Region((1, 0), (n0, n1 - 2), (2, 1))
    rb = wire.Region((0, 2), (n0 - 1, n1), (2, 1))
    shape = ra.shape()
    node = wire.Node(0, [
        wire.Ast(10, wire.OP_MUL, is_temp=True, shape=shape, operands=[(wire.scalar(3.0), None), (a_leaf, ra)]),
        wire.Ast(11, wire.OP_SUB, shape=shape, operands=[(wire.Ref(10), None), (b_leaf, rb)]),
    ])
    handle = ctx.compile_group(node)
    assert "in_str" in ctx.group_source(handle)
    A = torch.rand(n0, n1, dtype=torch.float64, device="cuda")
    B = torch.rand(n0, n1, dtype=torch.float64, device="cuda")
    out = torch.zeros(shape, dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    P = C.c_void_p
    ins = (P * 2)(A.data_ptr(), B.data_ptr())
    outs = (P * 1)(out.data_ptr())
    i64 = C.c_int64
    in_off = (i64 * 2)(1 * n1 + 0, 0 * n1 + 2)
    in_str = (i64 * 4)(2 * n1, 1, 2 * n1, 1)
    out_off = (i64 * 1)(0)
    out_str = (i64 * 2)(shape[1], 1)
    ext = (i64 * 2)(*shape)
    lib = _lib.load()
    _lib.check(ctx._h, lib.cn_launch_group(ctx._h, handle, 2, ins, in_off, in_str, 0, None, 1, outs,
                                           out_off, out_str, ext))
    ctx.synchronize()
    want = 3.0 * A[1::2, :n1 - 2] - B[0:n0 - 1:2, 2:]
    assert torch.equal(out, want)
