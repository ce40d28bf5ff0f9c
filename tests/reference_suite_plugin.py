"""pytest plugin for running the reference's own integration tests, unmodified, against this
package: it supplies the two fixtures those tests expect from their conftest (`interface`, and
the automatic reset of the frontend state) without starting any server.  The interface is the
oracle-backed stand-in unless CN_REFERENCE_SUITE_GPU=1 asks for the CUDA context."""
import os

import pytest


def pytest_configure(config):
    config.addinivalue_line("markers", "integration: the reference's marker for tests that need a backend")


@pytest.fixture(scope="session")
def interface():
    import charmnumeric_b200 as cnp
    if os.environ.get("CN_REFERENCE_SUITE_GPU") == "1":
        itf = cnp.CharmNumericInterface(device=0)
    else:
        from tests.helpers import OracleInterface
        itf = OracleInterface(dry_run=False)
    yield itf
    itf.close()


@pytest.fixture(autouse=True)
def _fresh_frontend():
    import charmnumeric_b200 as cnp
    cnp.reset_frontend_state()
    yield
    cnp.reset_frontend_state()
