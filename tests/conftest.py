import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle_mod():
    from oracle import oracle
    oracle.build()
    return oracle


@pytest.fixture(autouse=True)
def _fresh_frontend():
    """Mirror of the reference's autouse reset_frontend_state fixture (tests/conftest.py:135-141)."""
    import charmnumeric_b200 as cnp
    cnp.reset_frontend_state()
    yield
    cnp.reset_frontend_state()


@pytest.fixture(scope="session")
def interface():
    """One live backend context for the GPU tests (the reference's session fixture launches
    a LocalCluster, tests/conftest.py:144-186).  No GPU -> the context constructor raises:
    GPU tests never run on anything but the CUDA path."""
    import charmnumeric_b200 as cnp
    itf = cnp.CharmNumericInterface(device=int(os.environ.get("CN_TEST_DEVICE", "0")))
    yield itf
    itf.close()
