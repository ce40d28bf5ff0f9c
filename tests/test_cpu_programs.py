"""CPU-only: the oracle against the reference's known answers, and every GPU test program
pushed through the backend's host-side compiler (lowering + CUDA code generation + NVRTC for
sm_100a) without a GPU.

The known answers are the ones the reference's own tests and examples state
(tests/test_backend_integration.py:13-105, examples/cg.py:65-73, examples/matvec.py:45-55);
the reference keeps no golden files, every one of its checks is "the same expression in
NumPy", which is what is restated here.
"""
import numpy as np
import pytest

import charmnumeric_b200 as cnp
from charmnumeric_b200 import frontend as F
from tests import test_gpu_parity as G
from tests.helpers import DryRunOracle, OracleInterface


@pytest.fixture()
def cpu_interface():
    return OracleInterface(dry_run=True)


def test_reference_elementwise_expression(cpu_interface):
    G.test_elementwise_expression_roundtrip(cpu_interface)


@pytest.mark.parametrize("shape", [(8,), (4, 4), (4, 4, 4)])
def test_reference_elementwise_add(cpu_interface, shape):
    G.test_elementwise_add_roundtrip_all_ranks(cpu_interface, shape)


def test_reference_shifted_slices(cpu_interface):
    G.test_shifted_slice_expression_get_matches_numpy(cpu_interface)


def test_reference_strided_assignment(cpu_interface):
    G.test_strided_slice_assignment_roundtrip(cpu_interface)


def test_reference_jacobi3d_step(cpu_interface):
    G.test_jacobi3d_single_step_matches_numpy(cpu_interface)


def test_example_matvec_known_answer(cpu_interface):
    G.test_matvec_known_answer(cpu_interface)


def test_example_cg_dense(cpu_interface):
    G.test_cg_dense_matches_numpy_solve(cpu_interface)


@pytest.mark.parametrize("n,k", [(1, 0), (17, 0), (12, 2), (12, -3)])
def test_diag_through_the_oracle(cpu_interface, n, k):
    G.test_diag_matches_numpy(cpu_interface, n, k)


@pytest.mark.parametrize("shape,reps", [((5,), 3), ((7,), (4, 1)), ((3, 4), (2, 3)), ((2, 3, 4), (3, 1, 2))])
def test_tile_through_the_oracle(cpu_interface, shape, reps):
    G.test_tile_matches_numpy(cpu_interface, shape, reps)


def _dry(prog):
    cnp.reset_frontend_state()
    outs = prog()
    orc = DryRunOracle()
    F.execute(None, mirror=orc)
    return orc, outs


@pytest.mark.parametrize("prog", [
    G._jacobi2d_program(16, 64, 3),
    G._jacobi2d_program(33, 47, 4, res_every=2),
    G._jacobi3d_program((5, 7, 9), 2),
    G._jacobi3d_program((8, 8, 16), 2),
    G._cg_poisson_program(10, 3),
], ids=["jacobi2d", "jacobi2d_residual", "jacobi3d_odd", "jacobi3d_even", "cg"])
def test_gpu_programs_lower_and_compile(prog):
    orc, outs = _dry(prog)
    assert orc.compiled > 0
    for v in outs.values():
        assert np.all(np.isfinite(orc.get(v.name)))


def test_jacobi2d_interpreter_matches_c_loops(oracle_mod):
    """The numpy DAG interpreter and the threaded C restatement agree bit for bit."""
    n0, n1, iters = 40, 56, 10
    orc, outs = _dry(G._jacobi2d_program(n0, n1, iters, res_every=5))
    u = oracle_mod.randu((n0, n1), 0x5EED + 1)
    u[0, :] = 1.0
    u[-1, :] = 0.0
    u[:, 0] = 0.0
    u[:, -1] = 0.0
    scratch = np.zeros_like(u)
    res = np.zeros(2)
    oracle_mod.clib().cno_jacobi2d(oracle_mod._ptr(u), oracle_mod._ptr(scratch), n0, n1, 0.25, iters,
                                   5, oracle_mod._ptr(res), 16)
    assert orc.get(outs["u"].name).tobytes() == u.tobytes()
    np.testing.assert_allclose([orc.get(outs["res5"].name)[0], orc.get(outs["res10"].name)[0]],
                               res, rtol=1e-12)


def test_jacobi3d_interpreter_matches_c_loops(oracle_mod):
    shape, iters = (9, 12, 10), 4
    orc, outs = _dry(G._jacobi3d_program(shape, iters))
    u = oracle_mod.randu(shape, 0x5EED + 5)
    u[0] = 1.0
    u[-1] = 0.0
    u[:, 0] = 0.0
    u[:, -1] = 0.0
    u[:, :, 0] = 0.0
    u[:, :, -1] = 0.0
    scratch = np.zeros_like(u)
    oracle_mod.clib().cno_jacobi3d(oracle_mod._ptr(u), oracle_mod._ptr(scratch), *shape, 1.0 / 6.0,
                                   iters, 0, None, 4)
    assert orc.get(outs["u"].name).tobytes() == u.tobytes()


def test_chain_interpreter_matches_c(oracle_mod):
    n = 5000

    def prog():
        a = cnp.random.uniform((n,), seed=2, low=-1.0, high=1.0)
        b = cnp.random.uniform((n,), seed=3, low=-1.0, high=1.0)
        return {"r": G._chain(a, b), "s": cnp.sum(G._chain(a, b))}
    orc, outs = _dry(prog)
    a = oracle_mod.randu((n,), 2, -1, 1)
    b = oracle_mod.randu((n,), 3, -1, 1)
    out = np.empty(n)
    oracle_mod.clib().cno_chain_v(oracle_mod._ptr(a), oracle_mod._ptr(b), oracle_mod._ptr(out), n)
    assert orc.get(outs["r"].name).tobytes() == out.tobytes()
    s = oracle_mod.clib().cno_chain_sum(oracle_mod._ptr(a), oracle_mod._ptr(b), n, 0)
    assert abs(orc.get(outs["s"].name)[0] - s) <= 1e-12 * abs(s)


def test_cg_interpreter_matches_c_loops(oracle_mod):
    m, iters = 18, 6
    orc, outs = _dry(G._cg_poisson_program(m, iters))
    b = np.zeros((m, m))
    b[1:-1, 1:-1] = oracle_mod.randu((m, m), 0x5EED + 3)[1:-1, 1:-1]
    x, r, p, Ap = (np.zeros((m, m)) for _ in range(4))
    hist = np.zeros(iters)
    oracle_mod.clib().cno_cg_poisson(oracle_mod._ptr(b), oracle_mod._ptr(x), oracle_mod._ptr(r),
                                     oracle_mod._ptr(p), oracle_mod._ptr(Ap), m, iters,
                                     oracle_mod._ptr(hist), 64)
    np.testing.assert_allclose(orc.get(outs["x"].name), x, rtol=1e-11, atol=1e-14)
    np.testing.assert_allclose([orc.get(outs[f"rtr{k}"].name)[0] for k in range(iters)], hist,
                               rtol=1e-10)
    # CG on an SPD system: the residual norm has dropped
    assert hist[-1] < hist[0]


def test_exp_tanh_against_libm(oracle_mod):
    """The shared exp / tanh algorithm stays within a few ulp of this machine's libm."""
    rng = np.random.default_rng(7)
    x = np.concatenate([rng.uniform(-1, 0, 20000), rng.uniform(-700, 700, 20000),
                        rng.normal(0, 1e-3, 2000), [0.0, -0.0, 1e-300, 709.0, -744.0]])
    got, want = oracle_mod.exp(x), np.exp(x)
    ok = np.isfinite(want) & (want > 0)
    ulp = np.abs(got[ok] - want[ok]) / np.spacing(want[ok])
    assert ulp.max() <= 1.0
    assert np.isinf(oracle_mod.exp(np.array([710.0]))[0]) and oracle_mod.exp(np.array([-746.0]))[0] == 0.0
    assert np.isnan(oracle_mod.exp(np.array([np.nan]))[0])
    t = np.concatenate([rng.uniform(-3, 3, 20000), rng.normal(0, 1e-2, 5000), rng.uniform(-30, 30, 2000)])
    got, want = oracle_mod.tanh(t), np.tanh(t)
    nz = want != 0
    assert (np.abs(got[nz] - want[nz]) / np.spacing(np.abs(want[nz]))).max() <= 4.0


def test_seeded_generator_known_answers(oracle_mod):
    """First values of the counter-based generator (seed 0x5EED), pinned as text so that a
    change of the generator on either side is caught."""
    v = oracle_mod.randu((4,), 0x5EED)
    want = [float.fromhex(h) for h in GOLDEN_RANDU]
    assert v.tolist() == want
    # element g depends on (seed, g) only: a slab generated with an offset equals the slice
    whole = oracle_mod.randu((1000,), 99, -1.0, 1.0)
    part = oracle_mod.randu((300,), 99, -1.0, 1.0, offset=500)
    assert np.array_equal(whole[500:800], part)


GOLDEN_RANDU = None  # filled in below from tests/golden/randu_5eed.txt


def _load_golden():
    from pathlib import Path
    global GOLDEN_RANDU
    path = Path(__file__).parent / "golden" / "randu_5eed.txt"
    GOLDEN_RANDU = path.read_text().split()


_load_golden()


@pytest.mark.parametrize("n,tile,npe", [(40, 16, 3), (37, 8, 4), (33, 64, 2), (50, 7, 5)])
def test_tiled_jacobi2d_matches_the_flat_loops(oracle_mod, n, tile, npe):
    """The reference-structured timing variant (tiles as separate allocations, packed halo
    messages, result buffer + copy, one worker per PE) computes the very bits of the flat
    loops; the residuals differ by summation order only."""
    iters = 12
    u = oracle_mod.randu((n, n), 0x5EED + 1)
    u[0, :] = 1.0
    u[-1, :] = 0.0
    u[:, 0] = 0.0
    u[:, -1] = 0.0
    v = u.copy()
    scratch = np.zeros_like(u)
    res_flat, res_tiled = np.zeros(3), np.zeros(3)
    lib = oracle_mod.clib()
    lib.cno_jacobi2d(oracle_mod._ptr(u), oracle_mod._ptr(scratch), n, n, 0.25, iters, 5,
                     oracle_mod._ptr(res_flat), 16)
    secs = np.zeros(1)
    lib.cno_jacobi2d_tiled(oracle_mod._ptr(v), n, 0.25, iters, 5, oracle_mod._ptr(res_tiled), tile, npe,
                           oracle_mod._ptr(secs))
    assert v.tobytes() == u.tobytes()
    np.testing.assert_allclose(res_tiled[:2], res_flat[:2], rtol=1e-12)
    assert secs[0] >= 0.0


@pytest.mark.parametrize("m,tile,npe", [(18, 8, 3), (35, 16, 4), (34, 64, 1), (41, 5, 6)])
def test_tiled_cg_matches_the_flat_loops(oracle_mod, m, tile, npe):
    iters = 8
    b = np.zeros((m, m))
    b[1:-1, 1:-1] = oracle_mod.randu((m, m), 0x5EED + 3)[1:-1, 1:-1]
    x, r, p, Ap = (np.zeros((m, m)) for _ in range(4))
    hist, hist_t = np.zeros(iters), np.zeros(iters)
    lib = oracle_mod.clib()
    lib.cno_cg_poisson(oracle_mod._ptr(b), oracle_mod._ptr(x), oracle_mod._ptr(r), oracle_mod._ptr(p),
                       oracle_mod._ptr(Ap), m, iters, oracle_mod._ptr(hist), 64)
    xt = np.zeros((m, m))
    secs = np.zeros(1)
    lib.cno_cg_poisson_tiled(oracle_mod._ptr(b), oracle_mod._ptr(xt), m, iters, oracle_mod._ptr(hist_t), tile,
                             npe, oracle_mod._ptr(secs))
    # same operations on every point; only the order of the dot products' partial sums differs
    np.testing.assert_allclose(hist_t, hist, rtol=1e-10)
    np.testing.assert_allclose(xt, x, rtol=1e-10, atol=1e-14)
