"""GPU parity tests: every case runs one frontend program through the C ABI on the B200 and
through the CPU oracle on the very same DAG.  Elementwise / stencil / fill / copy results must
be bit-exact; reductions, matvec and CG iterates within 1e-10 relative (the tolerance the
backend is specified to; the reference's own reduction order is not fixed either).

The first block restates the reference's integration tests
(tests/test_backend_integration.py:13-105) against the same NumPy expressions.
"""
import numpy as np
import pytest

import charmnumeric_b200 as cnp
from tests.helpers import assert_bit_exact, assert_rel, run_both

pytestmark = pytest.mark.gpu

RTOL_REDUCTION = 1e-10


# ---- the reference's own integration cases ---------------------------------------------------

def test_elementwise_expression_roundtrip(interface):
    a = cnp.create_array((32,), dtype=np.float32)
    b = cnp.create_array((32,), dtype=np.float32)
    a[:] = 1.5
    b[:] = -0.5
    got = (2.0 * (a + b + 3.0)).get(interface)
    np.testing.assert_allclose(got, np.full((32,), 8.0, dtype=np.float32))


@pytest.mark.parametrize("shape", [(8,), (4, 4), (4, 4, 4)])
def test_elementwise_add_roundtrip_all_ranks(interface, shape):
    lhs = cnp.create_array(shape, dtype=np.float32)
    rhs = cnp.create_array(shape, dtype=np.float32)
    lhs[...] = 1.0
    rhs[...] = 1.0
    got = (lhs + rhs).get(interface)
    np.testing.assert_allclose(got, np.full(shape, 2.0, dtype=np.float32))


def test_shifted_slice_expression_get_matches_numpy(interface):
    src = cnp.arange(512, dtype=np.float32)
    got = (src[100:300] + src[150:350]).get(interface)
    host = np.arange(512, dtype=np.float32)
    np.testing.assert_allclose(got, host[100:300] + host[150:350])


def test_strided_slice_assignment_roundtrip(interface):
    n = 17
    coarse_n = (n - 1) // 2 + 1
    coarse = cnp.create_array((coarse_n, coarse_n), dtype=np.float64)
    fine = cnp.create_array((n, n), dtype=np.float64)
    coarse[:, :] = 0.0
    fine[:, :] = 1.0
    coarse[1:-1, 1:-1] = fine[2:-2:2, 2:-2:2]
    got = coarse.get(interface)
    want = np.zeros((coarse_n, coarse_n), dtype=np.float64)
    want[1:-1, 1:-1] = np.ones((n, n), dtype=np.float64)[2:-2:2, 2:-2:2]
    np.testing.assert_array_equal(got, want)


def test_jacobi3d_single_step_matches_numpy(interface):
    u = cnp.create_array((4, 4, 4), dtype=np.float32)
    u[0, :, :] = 1.0
    u[-1, :, :] = 1.0
    u[:, 0, :] = 1.0
    u[:, -1, :] = 1.0
    u[:, :, 0] = 1.0
    u[:, :, -1] = 1.0
    u[1:-1, 1:-1, 1:-1] = (1.0 / 6.0) * (
        u[:-2, 1:-1, 1:-1] + u[2:, 1:-1, 1:-1] + u[1:-1, :-2, 1:-1]
        + u[1:-1, 2:, 1:-1] + u[1:-1, 1:-1, :-2] + u[1:-1, 1:-1, 2:])
    got = u.get(interface)
    want = np.zeros((4, 4, 4), dtype=np.float32)
    want[0, :, :] = 1.0
    want[-1, :, :] = 1.0
    want[:, 0, :] = 1.0
    want[:, -1, :] = 1.0
    want[:, :, 0] = 1.0
    want[:, :, -1] = 1.0
    want[1:-1, 1:-1, 1:-1] = (1.0 / 6.0) * (
        want[:-2, 1:-1, 1:-1] + want[2:, 1:-1, 1:-1] + want[1:-1, :-2, 1:-1]
        + want[1:-1, 2:, 1:-1] + want[1:-1, 1:-1, :-2] + want[1:-1, 1:-1, 2:])
    np.testing.assert_allclose(got, want)


# ---- seeded parity against the oracle ---------------------------------------------------------

def _jacobi2d_program(n0, n1, iters, res_every=0):
    def prog():
        u = cnp.random.uniform((n0, n1), seed=0x5EED + 1)
        u[0, :] = 1.0
        u[-1, :] = 0.0
        u[:, 0] = 0.0
        u[:, -1] = 0.0
        out = {"u": u}
        for it in range(1, iters + 1):
            new = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:])
            if res_every and it % res_every == 0:
                d = new - u[1:-1, 1:-1]
                sq = d * d
                u[1:-1, 1:-1] = new
                out[f"res{it}"] = cnp.sum(sq)
                del d, sq
            else:
                u[1:-1, 1:-1] = new
            del new
        return out
    return prog


@pytest.mark.parametrize("shape", [(3, 3), (7, 7), (16, 64), (255, 255), (130, 258), (512, 512)])
def test_jacobi2d_bit_exact(interface, shape):
    gpu, cpu = run_both(interface, _jacobi2d_program(shape[0], shape[1], 5))
    assert_bit_exact(gpu, cpu)


def test_jacobi2d_residual_fused(interface):
    before = interface.context.stats()
    gpu, cpu = run_both(interface, _jacobi2d_program(256, 384, 10, res_every=5))
    after = interface.context.stats()
    assert_bit_exact({"u": gpu["u"]}, {"u": cpu["u"]})
    assert_rel({k: gpu[k] for k in ("res5", "res10")}, {k: cpu[k] for k in ("res5", "res10")},
               RTOL_REDUCTION)
    # 10 stencil groups (2 with the residual fused in) + uniform fill + 4 boundary fills
    assert after["group_launches"] - before["group_launches"] == 10


def test_jacobi2d_config1_full_size(interface):
    """BASELINE config 1 at full size: 2048 x 2048, 100 iterations, residual every 10."""
    gpu, cpu = run_both(interface, _jacobi2d_program(2048, 2048, 100, res_every=10))
    assert_bit_exact({"u": gpu["u"]}, {"u": cpu["u"]})
    keys = [f"res{i}" for i in range(10, 101, 10)]
    assert_rel({k: gpu[k] for k in keys}, {k: cpu[k] for k in keys}, RTOL_REDUCTION)


def _jacobi3d_program(shape, iters):
    def prog():
        u = cnp.random.uniform(shape, seed=0x5EED + 5)
        u[0, :, :] = 1.0
        u[-1, :, :] = 0.0
        u[:, 0, :] = 0.0
        u[:, -1, :] = 0.0
        u[:, :, 0] = 0.0
        u[:, :, -1] = 0.0
        c = 1.0 / 6.0
        for _ in range(iters):
            u[1:-1, 1:-1, 1:-1] = c * (u[:-2, 1:-1, 1:-1] + u[2:, 1:-1, 1:-1] + u[1:-1, :-2, 1:-1]
                                       + u[1:-1, 2:, 1:-1] + u[1:-1, 1:-1, :-2] + u[1:-1, 1:-1, 2:])
        return {"u": u}
    return prog


@pytest.mark.parametrize("shape", [(3, 3, 3), (5, 7, 9), (16, 16, 16), (33, 20, 64), (64, 48, 130)])
def test_jacobi3d_bit_exact(interface, shape):
    gpu, cpu = run_both(interface, _jacobi3d_program(shape, 3))
    assert_bit_exact(gpu, cpu)


def _chain(a, b):
    return cnp.exp(-a * a) * b + cnp.sqrt(cnp.abs(a)) - 0.5 * b * b + a / (1 + cnp.abs(b))


@pytest.mark.parametrize("n", [1, 2, 7, 255, 4096, 100003, 1 << 20])
def test_fused_chain_elementwise_bit_exact(interface, n):
    def prog():
        a = cnp.random.uniform((n,), seed=0x5EED + 2, low=-1.0, high=1.0)
        b = cnp.random.uniform((n,), seed=0x5EED + 3, low=-1.0, high=1.0)
        return {"a": a, "b": b, "r": _chain(a, b)}
    gpu, cpu = run_both(interface, prog)
    assert_bit_exact(gpu, cpu)


@pytest.mark.parametrize("n", [1, 255, 100003, 1 << 22])
def test_fused_chain_sum(interface, n):
    def prog():
        a = cnp.random.uniform((n,), seed=0x5EED + 2, low=-1.0, high=1.0)
        b = cnp.random.uniform((n,), seed=0x5EED + 3, low=-1.0, high=1.0)
        return {"s": cnp.sum(_chain(a, b))}
    before = interface.context.stats()
    gpu, cpu = run_both(interface, prog)
    after = interface.context.stats()
    assert_rel(gpu, cpu, RTOL_REDUCTION)
    # two fills + ONE fused kernel (expression and sum)
    assert after["kernel_launches"] - before["kernel_launches"] == 3
    # run-to-run bit reproducibility of the deterministic finish
    gpu2, _ = run_both(interface, prog)
    assert gpu2["s"].tobytes() == gpu["s"].tobytes()


@pytest.mark.parametrize("shape", [(1,), (1000,), (300, 7), (9, 10, 11), (1 << 21,)])
def test_dot_and_sum(interface, shape):
    def prog():
        a = cnp.random.uniform(shape, seed=11, low=-1.0, high=1.0)
        b = cnp.random.uniform(shape, seed=12, low=-1.0, high=1.0)
        return {"dot": cnp.dot2d(a, b), "sum": cnp.sum(a)}
    gpu, cpu = run_both(interface, prog)
    assert_rel(gpu, cpu, RTOL_REDUCTION)


@pytest.mark.parametrize("shape", [(1, 1), (48, 48), (37, 129), (256, 1000), (513, 2048)])
def test_matvec(interface, shape):
    def prog():
        A = cnp.random.uniform(shape, seed=21, low=-1.0, high=1.0)
        x = cnp.random.uniform((shape[1],), seed=22, low=-1.0, high=1.0)
        return {"y": A @ x}
    gpu, cpu = run_both(interface, prog)
    assert_rel(gpu, cpu, RTOL_REDUCTION)


def test_matvec_known_answer(interface):
    """examples/matvec.py:13-55: A[i, j] = i + j, x = 1."""
    M = N = 48
    host = np.add.outer(np.arange(M, dtype=np.float64), np.arange(N, dtype=np.float64))
    A = cnp.asarray(host)
    x = cnp.ones((N,), dtype=np.float64)
    got = A.matvec(x).get(interface)
    np.testing.assert_allclose(got, host @ np.ones(N))


@pytest.mark.parametrize("n,k", [(1, 0), (48, 0), (131, 0), (40, 3), (40, -5)])
def test_diag_matches_numpy(interface, n, k):
    """DIAG both ways (charmnumeric/operations.py:125-148): vector -> matrix, matrix -> vector."""
    v = np.arange(1.0, n + 1.0)
    m = np.arange(float((n + 2) * (n + 5))).reshape(n + 2, n + 5)
    built = cnp.diag(cnp.asarray(v), k).get(interface)
    assert np.array_equal(built, np.diag(v, k))
    taken = cnp.diag(cnp.asarray(m), k).get(interface)
    assert np.array_equal(taken, np.diag(m, k))
    tall = cnp.diag(cnp.asarray(np.ascontiguousarray(m.T)), k).get(interface)
    assert np.array_equal(tall, np.diag(m.T, k))


@pytest.mark.parametrize("shape,reps", [((5,), 3), ((7,), (4, 1)), ((3, 4), (2, 3)), ((6,), (2, 3, 2)),
                                        ((2, 3, 4), (3, 1, 2)), ((1,), (9,))])
def test_tile_matches_numpy(interface, shape, reps):
    """TILE (charmnumeric/operations.py:52-72), e.g. tile(h0, (b, 1)) of examples/lstm_forward.py:31."""
    host = np.arange(1.0, 1.0 + int(np.prod(shape))).reshape(shape)
    got = cnp.tile(cnp.asarray(host), reps).get(interface)
    assert np.array_equal(got, np.tile(host, reps))


def _cg_poisson_program(m, iters):
    def prog():
        b = cnp.zeros((m, m))
        b[1:-1, 1:-1] = cnp.random.uniform((m, m), seed=0x5EED + 3)[1:-1, 1:-1]
        x = cnp.zeros((m, m))
        r = b.copy()
        p = b.copy()
        Ap = cnp.zeros((m, m))
        rtr = cnp.dot2d(r, r)
        out = {}
        for k in range(iters):
            Ap[1:-1, 1:-1] = (4.0 * p[1:-1, 1:-1] - p[:-2, 1:-1] - p[2:, 1:-1]
                              - p[1:-1, :-2] - p[1:-1, 2:])
            pAp = cnp.dot2d(p, Ap)
            alpha = rtr / pAp
            x = x + alpha * p
            r = r - alpha * Ap
            rtr_new = cnp.dot2d(r, r)
            beta = rtr_new / rtr
            p = r + beta * p
            rtr = rtr_new
            out[f"rtr{k}"] = rtr
        out["x"] = x
        out["r"] = r
        return out
    return prog


@pytest.mark.parametrize("m,iters", [(10, 5), (66, 20), (258, 40)])
def test_cg_poisson_iterates(interface, m, iters):
    before = interface.context.stats()
    gpu, cpu = run_both(interface, _cg_poisson_program(m, iters))
    after = interface.context.stats()
    assert_rel(gpu, cpu, RTOL_REDUCTION)
    # both dots of every iteration ride in a group kernel
    assert after["fused_reductions"] - before["fused_reductions"] >= 2 * iters


def test_cg_dense_matches_numpy_solve(interface):
    """examples/cg.py:14-73: A = ones + N*I, b = 1..N, compared with numpy.linalg.solve."""
    N = 128
    A_np = np.ones((N, N)) + N * np.eye(N)
    b_np = np.arange(1, N + 1, dtype=np.float64)
    A = cnp.asarray(A_np)
    b = cnp.asarray(b_np)
    x = cnp.zeros((N,))
    r = b.copy()
    p = b.copy()
    rtr = r @ r
    for _ in range(4):
        Ap = A @ p
        pAp = p @ Ap
        alpha = rtr / pAp
        x = x + alpha * p
        r = r - alpha * Ap
        rtr_new = r @ r
        beta = rtr_new / rtr
        p = r + beta * p
        rtr = rtr_new
    got = x.get(interface)
    assert np.allclose(got, np.linalg.solve(A_np, b_np))


def test_power_iteration(interface):
    """examples/reduction.py:5-6 with the sqrt addition: y = A x; x = y / sqrt(y.y)."""
    n = 512

    def prog():
        A = cnp.random.uniform((n, n), seed=0x5EED + 4, low=-1.0 / 256, high=1.0 / 256)
        x = cnp.random.uniform((n,), seed=0x5EED + 44, low=-1.0, high=1.0)
        for _ in range(5):
            y = A @ x
            s = y @ y
            x = y / cnp.sqrt(s)
        return {"x": x, "s": s}
    gpu, cpu = run_both(interface, prog)
    assert_rel(gpu, cpu, 1e-9)


# ---- strided / sub-region groups, other dtypes ----------------------------------------------------

def test_restriction_and_red_black(interface):
    def prog():
        n = 33
        fine = cnp.random.uniform((n, n), seed=31)
        coarse = cnp.zeros(((n - 1) // 2 + 1,) * 2)
        coarse[1:-1, 1:-1] = 0.25 * fine[2:-2:2, 2:-2:2] + 0.125 * (
            fine[1:-3:2, 2:-2:2] + fine[3:-1:2, 2:-2:2] + fine[2:-2:2, 1:-3:2] + fine[2:-2:2, 3:-1:2])
        u = cnp.random.uniform((n, n), seed=32)
        # red points of a Gauss-Seidel sweep (examples/gauss_seidel.py:30-54)
        u[1:-1:2, 1:-1:2] = 0.25 * (u[0:-2:2, 1:-1:2] + u[2::2, 1:-1:2]
                                    + u[1:-1:2, 0:-2:2] + u[1:-1:2, 2::2])
        return {"coarse": coarse, "u": u}
    gpu, cpu = run_both(interface, prog)
    assert_bit_exact(gpu, cpu)


def test_row_copy_hazard_small_region(interface):
    def prog():
        u = cnp.random.uniform((64, 50), seed=41)
        u[0, :] = u[1, :]
        u[:, 0] = u[:, 1]
        u[1:5, 2:9] = u[0:4, 1:8]
        return {"u": u}
    gpu, cpu = run_both(interface, prog)
    assert_bit_exact(gpu, cpu)


@pytest.mark.parametrize("dtype", [np.float32, np.int32, np.int64])
def test_other_dtypes(interface, dtype):
    def prog():
        a = cnp.asarray(np.arange(1, 1001).astype(dtype))
        b = cnp.asarray((np.arange(1000) % 7 + 1).astype(dtype))
        c = (a + b) * 3 - a / b
        return {"c": c, "d": cnp.dot2d(a, b)}
    gpu, cpu = run_both(interface, prog)
    if np.dtype(dtype).kind == "f":
        assert_rel(gpu, cpu, 1e-6)
    else:
        assert_bit_exact(gpu, cpu)


def test_tanh_exp_bit_exact(interface):
    def prog():
        a = cnp.random.uniform((50001,), seed=51, low=-6.0, high=6.0)
        return {"t": cnp.tanh(a), "e": cnp.exp(a * 100.0)}
    gpu, cpu = run_both(interface, prog)
    assert_bit_exact(gpu, cpu)


# ---- error behaviour: status codes instead of aborts ------------------------------------------------

def test_error_codes(interface):
    from charmnumeric_b200 import wire
    from charmnumeric_b200._lib import CnError
    ctx = interface.context
    with pytest.raises(CnError) as e:
        ctx.receive_dag(b"nonsense-not-a-blob")
    assert e.value.status == 2
    missing = wire.Node(0, [wire.Ast(900001, wire.OP_ADD, shape=(8,), operands=[
        (wire.leaf(900002, (8,)), None), (wire.leaf(900003, (8,)), None)])])
    with pytest.raises(CnError) as e:
        ctx.run([missing])
    assert e.value.status == 3
    bad_op = wire.Node(0, [wire.Ast(900004, 77, shape=(8,))], fusible=False)
    with pytest.raises(CnError) as e:
        ctx.run([bad_op])
    assert e.value.status == 6
    with pytest.raises(CnError) as e:
        ctx.get(987654, (4,), np.float64)
    assert e.value.status == 3
    # the context stays usable after errors
    a = cnp.ones((16,))
    assert np.array_equal((a + a).get(interface), np.full(16, 2.0))


def test_bounded_device_wait_reports_status(interface):
    """Failure path of the staged stencil kernels, without faulting or hanging anything: with
    the test hook on, the elected thread issues no tile copy, every consumer's bounded wait runs
    out, the kernel leaves, and the next synchronise reports it as a status code.  The context
    stays usable."""
    from charmnumeric_b200._lib import CnError
    ctx = interface.context
    prog = _jacobi2d_program(64, 256, 1)
    try:
        ctx.set_option("staged", 2)
        ctx.set_option("debug_drop_copies", 1)
        cnp.reset_frontend_state()
        outs = prog()
        with pytest.raises(CnError) as e:
            outs["u"].get(interface)
        assert e.value.status == 8 and "gave up waiting" in e.value.message
    finally:
        ctx.set_option("debug_drop_copies", 0)
        ctx.set_option("staged", 1)
    gpu, cpu = run_both(interface, prog)
    assert_bit_exact(gpu, cpu)


def test_bounded_peer_wait_reports_status(interface):
    """Failure path of the cross-GPU transport on one GPU: a halo exchange against a scratch
    mailbox whose partner never answers.  The kernel's bounded wait runs out, it sets the error
    word and returns; the next synchronise reports a status code and the context stays usable."""
    from charmnumeric_b200._lib import CnError
    ctx = interface.context
    ctx.synchronize()
    ctx.set_option("debug_peer_wait", 1)
    with pytest.raises(CnError) as e:
        ctx.synchronize()
    assert e.value.status == 8 and "another GPU" in e.value.message
    ctx.synchronize()
    a = cnp.ones((32,))
    assert np.array_equal((a + a).get(interface), np.full(32, 2.0))


def test_rank_marked_failed_stops_collective_work():
    """Host-side failure notice: once a rank is marked failed, DAG submission returns
    CN_STATUS_RANK_FAILED instead of enqueuing work that would wait for that rank."""
    from charmnumeric_b200._lib import CnError
    ctx = cnp.Context(device=0)
    try:
        ctx.run([])
        ctx.mark_rank_failed(0)
        with pytest.raises(CnError) as e:
            ctx.run([])
        assert e.value.status == 14
    finally:
        ctx.close()


# ---- producer inlining: a whole-array assignment folded into the stencil behind it -----------

def _cg_rotated_program(m0, m1, iters):
    """CG entered at the direction update, the order the benchmark's step uses."""
    def prog():
        b = cnp.zeros((m0, m1))
        b[1:-1, 1:-1] = cnp.random.uniform((m0, m1), seed=0x5EED + 3)[1:-1, 1:-1]
        x = cnp.zeros((m0, m1))
        r = b.copy()
        p = b.copy()
        Ap = cnp.zeros((m0, m1))
        rtr = cnp.dot2d(r, r)
        beta = cnp.zeros((1,))
        out = {}
        for k in range(iters):
            p[...] = r + beta * p
            Ap[1:-1, 1:-1] = (4.0 * p[1:-1, 1:-1] - p[:-2, 1:-1] - p[2:, 1:-1]
                              - p[1:-1, :-2] - p[1:-1, 2:])
            pAp = cnp.dot2d(p, Ap)
            alpha = rtr / pAp
            x[...] = x + alpha * p
            r[...] = r - alpha * Ap
            rtr_new = cnp.dot2d(r, r)
            beta[...] = rtr_new / rtr
            rtr[...] = rtr_new
            out[f"rtr{k}"] = rtr_new
        out.update({"x": x, "r": r, "p": p, "Ap": Ap})
        return out
    return prog


@pytest.mark.parametrize("shape,iters", [((10, 10), 4), ((66, 130), 12), ((258, 258), 25)])
def test_cg_direction_update_inlined_into_stencil(interface, shape, iters):
    before = interface.context.stats()
    gpu, cpu = run_both(interface, _cg_rotated_program(shape[0], shape[1], iters))
    after = interface.context.stats()
    assert_rel(gpu, cpu, RTOL_REDUCTION)
    assert after["inlined_producers"] - before["inlined_producers"] == iters
    # one iteration = (p, Ap, p.Ap) + (x, r, r.r) + one size-1 kernel
    assert after["fused_reductions"] - before["fused_reductions"] >= 2 * iters


def test_inlined_producer_is_bit_exact(interface):
    """One direction update + stencil from seeded data: p and Ap must carry the very bits the
    two separate kernels (and the oracle) produce, on every shape class of tile."""
    for shape in [(7, 9), (64, 64), (131, 258), (40, 20, 34)]:
        def prog():
            nd = len(shape)
            r = cnp.random.uniform(shape, seed=71, low=-1.0, high=1.0)
            p = cnp.random.uniform(shape, seed=72, low=-1.0, high=1.0)
            beta = cnp.random.uniform((1,), seed=73)
            Ap = cnp.zeros(shape)
            p[...] = r + beta * p
            if nd == 2:
                Ap[1:-1, 1:-1] = (4.0 * p[1:-1, 1:-1] - p[:-2, 1:-1] - p[2:, 1:-1]
                                  - p[1:-1, :-2] - p[1:-1, 2:])
            else:
                Ap[1:-1, 1:-1, 1:-1] = (6.0 * p[1:-1, 1:-1, 1:-1] - p[:-2, 1:-1, 1:-1] - p[2:, 1:-1, 1:-1]
                                        - p[1:-1, :-2, 1:-1] - p[1:-1, 2:, 1:-1]
                                        - p[1:-1, 1:-1, :-2] - p[1:-1, 1:-1, 2:])
            return {"p": p, "Ap": Ap, "pAp": cnp.dot2d(p, Ap)}
        before = interface.context.stats()
        gpu, cpu = run_both(interface, prog)
        after = interface.context.stats()
        assert after["inlined_producers"] - before["inlined_producers"] == 1, shape
        assert_bit_exact({k: gpu[k] for k in ("p", "Ap")}, {k: cpu[k] for k in ("p", "Ap")})
        assert_rel({"pAp": gpu["pAp"]}, {"pAp": cpu["pAp"]}, RTOL_REDUCTION)


def test_producer_not_inlined_when_the_stencil_overwrites_its_input(interface):
    """`p = r + beta p` followed by a stencil that assigns into r: the pair must stay two
    kernels (the stencil's writes would feed back into the recomputed p), and stay correct."""
    def prog():
        r = cnp.random.uniform((33, 40), seed=81)
        p = cnp.random.uniform((33, 40), seed=82)
        beta = cnp.random.uniform((1,), seed=83)
        p[...] = r + beta * p
        r[1:-1, 1:-1] = 0.25 * (p[:-2, 1:-1] + p[2:, 1:-1] + p[1:-1, :-2] + p[1:-1, 2:])
        return {"p": p, "r": r}
    before = interface.context.stats()
    gpu, cpu = run_both(interface, prog)
    after = interface.context.stats()
    assert after["inlined_producers"] == before["inlined_producers"]
    assert_bit_exact(gpu, cpu)


# ---- cross-dimension SET_REGION (src/executor_transfer.cpp:66-177) ------------------------------

def _cross_dimension_program():
    A = cnp.random.uniform((37, 22), seed=61)
    v = cnp.random.uniform((22,), seed=62)
    c = cnp.random.uniform((37,), seed=63)
    w = cnp.zeros((37,))
    row = cnp.zeros((22,))
    A[5, :] = v                 # 1-D into a row
    A[:, 3] = c                 # 1-D into a column
    w[:] = A[:, 7]              # a column into 1-D
    row[:] = A[30, :]           # a row into 1-D
    H = cnp.zeros((6, 37, 22))
    H[2, :, 4:] = A[:, 4:]      # 2-D into a plane of a 3-D array (examples/lstm_forward.py:36)
    B = cnp.zeros((37, 22))
    B[1:36:2, :] = H[2, 1:36:2, :]   # a stepped plane back into 2-D
    col = cnp.zeros((37, 1))
    col[:, :] = c               # (n,) into (n, 1)
    return {"A": A, "w": w, "row": row, "H": H, "B": B, "col": col}


def test_cross_dimension_assignment(interface):
    gpu, cpu = run_both(interface, _cross_dimension_program)
    assert_bit_exact(gpu, cpu)


def test_cross_dimension_assignment_rejects_mismatched_shapes():
    a = cnp.zeros((5, 6))
    v = cnp.zeros((5,))
    with pytest.raises(ValueError):
        a[2, :] = v
