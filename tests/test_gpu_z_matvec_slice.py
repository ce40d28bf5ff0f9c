"""Matvec on views of the matrix and the vector (the cases of the reference's
examples/matvec_slice.py:27-92: full, row slice, column slice, both, offsets that are not
multiples of any tile size), against NumPy."""
import numpy as np
import pytest

import charmnumeric_b200 as cnp

pytestmark = pytest.mark.gpu

M = N = 128
CASES = [((0, M), (0, N)), ((0, 32), (0, N)), ((0, M), (16, 48)), ((8, 40), (10, 50)), ((3, 37), (5, 47))]


@pytest.mark.parametrize("rows,cols", CASES)
def test_matvec_on_slices(interface, rows, cols):
    rng = np.random.default_rng(7)
    A_np = rng.uniform(-1.0, 1.0, (M, N))
    x_np = np.arange(1.0, N + 1.0)
    A = cnp.asarray(A_np)
    x = cnp.asarray(x_np)
    (r0, r1), (c0, c1) = rows, cols
    got = A[r0:r1, c0:c1].matvec(x[c0:c1]).get(interface)
    want = A_np[r0:r1, c0:c1] @ x_np[c0:c1]
    assert got.shape == want.shape
    assert np.max(np.abs(got - want)) <= 1e-10 * np.max(np.abs(want))


def test_matvec_with_a_column_vector(interface):
    """examples/matvec.py:30-34 (default mode): the vector is an (n, 1) column, the result (m, 1)."""
    rng = np.random.default_rng(11)
    A_np = rng.uniform(-1.0, 1.0, (48, 64))
    x_np = rng.uniform(-1.0, 1.0, (64, 1))
    got = cnp.asarray(A_np).matvec(cnp.asarray(x_np)).get(interface)
    want = A_np @ x_np
    assert got.shape == (48, 1)
    assert np.max(np.abs(got - want)) <= 1e-10 * np.max(np.abs(want))
