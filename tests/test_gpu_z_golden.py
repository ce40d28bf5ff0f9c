"""The committed golden vectors (tests/golden/reference_kats.npz: what the reference's own tests
and examples compare against) through the CUDA path: the same test bodies as
tests/test_oracle_golden.py, run against the GPU interface instead of the oracle."""
import pytest

from tests import test_oracle_golden as T

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("body", [T.test_expression, T.test_shifted_slices, T.test_strided_assignment,
                                  T.test_jacobi3d_step_is_a_true_jacobi_step, T.test_cg_dense_solution,
                                  T.test_matvec_i_plus_j, T.test_diag_matrix_extract],
                         ids=lambda f: f.__name__[5:])
def test_golden_vector(interface, body):
    body(interface)


@pytest.mark.parametrize("k", [0, 1, -1])
def test_golden_diag_vector(interface, k):
    T.test_diag_vector(interface, k)
