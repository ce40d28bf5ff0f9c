"""The seeded random programs of tests/test_frontend_fuzz.py on the CUDA path: every array the
GPU produces must be bit-identical to NumPy's eager evaluation of the same program (only
IEEE-exact operations are generated: +, -, *, /, abs, sqrt; division and square root are
compiled IEEE-rounded), reductions and matvec within 1e-10.  A mismatch fails the suite, with
the seed in the message."""
import pytest

import charmnumeric_b200 as cnp
from tests import test_frontend_fuzz as T

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", [3, 4, 5, 6, 8, 13, 16, 21, 1001, 1003, 1004, 1006])
def test_random_program_on_the_gpu(interface, seed):
    cnp.reset_frontend_state()
    T._program(seed, interface)
