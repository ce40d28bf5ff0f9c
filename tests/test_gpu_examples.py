"""The example programs (ports of the reference's examples/*.py to this package) run to
completion on the GPU and pass their own self-checks."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("script,args", [
    ("jacobi2d.py", ["256", "20"]),
    ("jacobi3d.py", ["48", "20"]),
    ("cg.py", ["128", "4"]),
    ("matvec.py", ["48"]),
    ("gauss_seidel.py", ["130", "6"]),
    ("multigrid2d.py", ["65", "2"]),
    ("jacobi_iteration.py", ["96", "50"]),
])
def test_example_runs(script, args):
    env_path = str(ROOT)
    res = subprocess.run([sys.executable, str(ROOT / "examples" / script)] + args, capture_output=True,
                         text=True, timeout=300, env={**__import__("os").environ, "PYTHONPATH": env_path})
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
