"""CPU-only: the oracle against the committed golden vectors (tests/golden/reference_kats.npz,
made by tests/golden/make_golden.py from the expressions the reference's own tests and examples
check against: tests/test_backend_integration.py:13-127, examples/cg.py:65-73,
examples/matvec.py:45-55)."""
from pathlib import Path

import numpy as np
import pytest

import charmnumeric_b200 as cnp
from tests.helpers import OracleInterface

GOLDEN = np.load(Path(__file__).parent / "golden" / "reference_kats.npz")


@pytest.fixture()
def itf():
    return OracleInterface(dry_run=False)


def test_expression(itf):
    a = cnp.create_array((32,), dtype=np.float32)
    b = cnp.create_array((32,), dtype=np.float32)
    a[:] = 1.5
    b[:] = -0.5
    got = (2.0 * (a + b + 3.0)).get(itf)
    assert got.dtype == np.float32 and np.array_equal(got, GOLDEN["expr_f32"])


def test_shifted_slices(itf):
    src = cnp.arange(512, dtype=np.float32)
    assert np.array_equal((src[100:300] + src[150:350]).get(itf), GOLDEN["shifted_f32"])


def test_strided_assignment(itf):
    coarse = cnp.create_array((9, 9), dtype=np.float64)
    fine = cnp.create_array((17, 17), dtype=np.float64)
    coarse[:, :] = 0.0
    fine[:, :] = 1.0
    coarse[1:-1, 1:-1] = fine[2:-2:2, 2:-2:2]
    assert np.array_equal(coarse.get(itf), GOLDEN["strided_f64"])


def test_jacobi3d_step_is_a_true_jacobi_step(itf):
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
    np.testing.assert_allclose(u.get(itf), GOLDEN["jacobi3d_f32"], rtol=1e-7)


def test_cg_dense_solution(itf):
    N = 128
    A = cnp.asarray(np.ones((N, N)) + N * np.eye(N))
    b = cnp.asarray(np.arange(1, N + 1, dtype=np.float64))
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
    assert np.allclose(x.get(itf), GOLDEN["cg_solution"])


def test_matvec_i_plus_j(itf):
    M = 48
    A = cnp.asarray(np.add.outer(np.arange(M, dtype=np.float64), np.arange(M, dtype=np.float64)))
    x = cnp.ones((M,), dtype=np.float64)
    assert np.allclose(A.matvec(x).get(itf), GOLDEN["matvec_ipj"])


@pytest.mark.parametrize("k", [0, 1, -1])
def test_diag_vector(itf, k):
    """tests/test_backend_integration.py:108-116."""
    vector = cnp.create_array((8,), dtype=np.float64)
    vector[:] = 2.0
    assert np.array_equal(cnp.diag(vector, k=k).get(itf), GOLDEN[f"diag_vector_k{k}"])


def test_diag_matrix_extract(itf):
    """tests/test_backend_integration.py:119-127."""
    matrix = cnp.create_array((6, 10), dtype=np.float64)
    matrix[:, :] = 3.0
    assert np.array_equal(cnp.diag(matrix, k=2).get(itf), GOLDEN["diag_matrix_k2"])
