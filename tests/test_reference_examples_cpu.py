"""The reference's own example programs, unmodified, through the import shims
(charmnumeric_b200/compat: ``import charmnumeric``, ``from charmtyles.core import execute``).

Runs where a checkout of the reference sits beside this repository (or where
CHARMNUMERIC_REFERENCE points to one) and is skipped elsewhere.  There is no GPU in this test:
the programs build their DAGs with the real frontend, and the interface they connect to is
the oracle-backed stand-in, so what is checked is the frontend (API coverage, grouping, wire
nodes) against each program's own NumPy self-check."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REFERENCE = Path(os.environ.get("CHARMNUMERIC_REFERENCE", ROOT.parent / "reference"))
EXAMPLES = REFERENCE / "examples"

BOOTSTRAP = """
import runpy, sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {compat!r})
import charmnumeric, charmnumeric_b200
from tests.helpers import OracleInterface
make = lambda *a, **k: OracleInterface(dry_run=False)
charmnumeric.CharmNumericInterface = make
charmnumeric_b200.CharmNumericInterface = make
sys.argv = sys.argv[1:]
runpy.run_path(sys.argv[0], run_name="__main__")
"""

# program, extra arguments, text its own self-check prints on success (None: runs to completion)
PROGRAMS = [
    ("simple.py", [], None),
    ("reduction.py", [], None),
    ("jacobi.py", [], None),
    ("jacobi2d.py", [], None),
    ("jacobi3d.py", [], None),
    ("test.py", [], None),                       # asserts array_equal itself
    ("diag.py", [], "All tests passed!"),
    ("cg.py", [], "Match: True"),
    ("matvec.py", [], "Match: True"),            # (n, 1) column vector
    ("matvec.py", ["--cross"], "Match: True"),   # 1-D vector
    ("jacobi_iteration.py", [], "Converged   = True"),
    ("gauss_seidel.py", [], None),
    ("multigrid2d.py", [], "V-cycle 10"),
]


@pytest.mark.skipif(not EXAMPLES.is_dir(), reason="no checkout of the reference next to this repository")
@pytest.mark.parametrize("program,args,expect", PROGRAMS, ids=[p + "".join(a) for p, a, _ in PROGRAMS])
def test_reference_example_runs_unmodified(program, args, expect):
    code = BOOTSTRAP.format(root=str(ROOT), compat=str(ROOT / "charmnumeric_b200" / "compat"))
    res = subprocess.run([sys.executable, "-c", code, str(EXAMPLES / program)] + args, capture_output=True,
                         text=True, timeout=600, cwd=str(ROOT))
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    if expect:
        assert expect in res.stdout, res.stdout[-1500:]


@pytest.mark.skipif(not (REFERENCE / "tests" / "test_backend_integration.py").is_file(),
                    reason="no checkout of the reference next to this repository")
def test_reference_integration_suite_runs_unmodified(tmp_path):
    """The reference's tests/test_backend_integration.py as it stands (its conftest, which starts
    a charmrun server, is left out; tests/reference_suite_plugin.py supplies the two fixtures)."""
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT), str(ROOT / "charmnumeric_b200" / "compat")])
    res = subprocess.run([sys.executable, "-m", "pytest", "--noconftest", "-p", "tests.reference_suite_plugin",
                          "-p", "no:cacheprovider", "-q", str(REFERENCE / "tests" / "test_backend_integration.py")],
                         capture_output=True, text=True, timeout=600, cwd=str(tmp_path), env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-1500:]
    assert " passed" in res.stdout and "failed" not in res.stdout
