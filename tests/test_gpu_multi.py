"""Multi-GPU parity: one process per GPU (slab partition; halo rows and reduction totals travel
through the peer mailboxes over NVLink, or through NCCL send/recv and allreduce when the peer
path is switched off), each rank fetches the whole result and compares it with the oracle that
ran the same DAG.  Needs at least two GPUs; skipped otherwise."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _gpu_count():
    import torch
    return torch.cuda.device_count()


def _run_ranks(tmp_path, case, nranks, p2p, overlap=0, halo=1, push=0):
    idfile = str(tmp_path / "nccl_id")
    env = dict(os.environ, CN_P2P=str(p2p), CN_OVERLAP_HALO=str(overlap), CN_HALO=str(halo), CN_PUSH_HALO=str(push))
    procs = [subprocess.Popen([sys.executable, str(ROOT / "tests" / "multi_worker.py"), str(r), str(nranks),
                               idfile, str(tmp_path), case], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True, env=env) for r in range(nranks)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outputs.append(out)
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} failed:\n{outputs[r][-3000:]}"
    return [np.load(tmp_path / f"{case}_rank{r}.npz") for r in range(nranks)]


def _check(case, results, p2p):
    exact = case.startswith("jacobi") or case == "tile"
    for r, d in enumerate(results):
        for key in d.files:
            if not key.startswith("gpu_"):
                continue
            g, c = d[key], d["cpu_" + key[4:]]
            if g.size > 1 and (exact or (case == "chain" and key == "gpu_r")):
                assert g.tobytes() == c.tobytes(), (case, r, key)
            else:
                scale = np.max(np.abs(c)) or 1.0
                assert np.max(np.abs(g - c)) <= 1e-10 * scale, (case, r, key)
        if case in ("jacobi2d", "jacobi3d", "cg"):
            assert int(d["halo_exchanges"]) > 0
        if case in ("jacobi2d", "jacobi3d", "cg", "chain"):
            # the peer path was really taken (or really not)
            assert (int(d["peer_exchanges"]) > 0) == bool(p2p), (case, r)
    # reduction results are summed in rank order on every rank: identical bits everywhere
    if p2p:
        for key in results[0].files:
            if key.startswith("gpu_") and results[0][key].size == 1:
                for d in results[1:]:
                    assert d[key].tobytes() == results[0][key].tobytes(), (case, key)


@pytest.mark.parametrize("case", ["jacobi2d", "jacobi2d_small", "jacobi3d", "cg", "chain", "matvec", "diag", "tile"])
@pytest.mark.parametrize("nranks", [2, 4])
def test_multi_gpu_matches_oracle(tmp_path, case, nranks):
    if _gpu_count() < nranks:
        pytest.skip(f"needs {nranks} GPUs")
    _check(case, _run_ranks(tmp_path, case, nranks, 1), 1)


@pytest.mark.parametrize("nranks,p2p", [(2, 1), (2, 0), (4, 1)])
def test_multi_gpu_stepped_views_across_slabs(tmp_path, nranks, p2p):
    """A multigrid V-cycle and red-black Gauss-Seidel sweeps: restriction, prolongation and the
    coloured sweeps read and write every second row, so operand rows travel between ranks."""
    if _gpu_count() < nranks:
        pytest.skip(f"needs {nranks} GPUs")
    results = _run_ranks(tmp_path, "multigrid", nranks, p2p)
    for r, d in enumerate(results):
        for key in ("u", "g"):
            assert d["gpu_" + key].tobytes() == d["cpu_" + key].tobytes(), (r, key)
        assert int(d["row_fetches"]) > 0


@pytest.mark.parametrize("nranks", [2, 4])
def test_multi_gpu_cross_dimension_assignment(tmp_path, nranks):
    """Rows into columns, columns into vectors, planes of a 3-D array: the source region is
    either row-aligned with the target or gathered onto every rank."""
    if _gpu_count() < nranks:
        pytest.skip(f"needs {nranks} GPUs")
    results = _run_ranks(tmp_path, "xset", nranks, 1)
    for r, d in enumerate(results):
        for key in d.files:
            if key.startswith("gpu_"):
                assert d[key].tobytes() == d["cpu_" + key[4:]].tobytes(), (r, key)


@pytest.mark.parametrize("nranks", [2, 4])
def test_multi_gpu_cg_direction_update_inlined(tmp_path, nranks):
    """CG entered at the direction update: the fused kernel reads r and p one row beyond the
    slab, both halos travel in one exchange."""
    if _gpu_count() < nranks:
        pytest.skip(f"needs {nranks} GPUs")
    results = _run_ranks(tmp_path, "cg_rotated", nranks, 1)
    _check("cg", results, 1)
    for d in results:
        assert int(d["inlined_producers"]) == 9


@pytest.mark.parametrize("case,halo", [("jacobi2d", 1), ("jacobi3d", 1), ("cg_rotated", 1), ("jacobi2d_long", 4)])
def test_multi_gpu_edge_rows_pushed_by_their_producers(tmp_path, case, halo):
    """Option push_halo: after the first exchange the kernels that rewrite an array store its
    edge rows into the neighbours' mailboxes themselves; a small kernel publishes them, waits
    for the neighbours' and copies those in.  Same results, bit for bit."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    results = _run_ranks(tmp_path, case, 2, 1, halo=halo, push=1)
    _check("cg" if case == "cg_rotated" else case.replace("_long", ""), results, 1)
    for d in results:
        assert int(d["halo_pushes"]) > 0


@pytest.mark.parametrize("case", ["jacobi2d", "jacobi3d", "cg", "chain"])
def test_multi_gpu_nccl_transport(tmp_path, case):
    """The same programs with the peer mailboxes switched off: NCCL moves halos and totals."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    _check(case, _run_ranks(tmp_path, case, 2, 0), 0)


@pytest.mark.parametrize("case", ["jacobi2d", "jacobi3d"])
def test_multi_gpu_overlapped_halo(tmp_path, case):
    """Option overlap_halo: sweeps without a fused reduction are cut along dimension 0 and the
    interior runs on the main stream beside the halo exchange and the edge rows."""
    if _gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    results = _run_ranks(tmp_path, case, 2, 1, overlap=1)
    _check(case, results, 1)
    for d in results:
        assert int(d["overlapped_sweeps"]) > 0


@pytest.mark.parametrize("case,halo,p2p,nranks", [
    ("jacobi2d_long", 4, 1, 2), ("jacobi2d_long", 3, 0, 2), ("jacobi3d_long", 4, 1, 2), ("cg", 4, 1, 2),
    ("jacobi3d_long", 2, 1, 2), ("jacobi2d_long", 4, 1, 4), ("jacobi3d_long", 2, 1, 4),
    ("jacobi2d_pingpong", 4, 1, 2), ("jacobi2d_pingpong", 4, 0, 2), ("jacobi2d_long", 16, 1, 2),
    ("jacobi2d_deep", 32, 1, 2), ("jacobi2d_deep", 64, 1, 2), ("jacobi2d_deep", 64, 1, 4),
    ("cg_rotated", 4, 1, 2)])
def test_multi_gpu_deep_halo(tmp_path, case, halo, p2p, nranks):
    """Halo depth above the stencil's reach: sweeps also update halo rows (redundantly with the
    neighbour), so one exchange serves several sweeps.  Results stay bit-exact."""
    if _gpu_count() < nranks:
        pytest.skip(f"needs {nranks} GPUs")
    results = _run_ranks(tmp_path, case, nranks, p2p, halo=halo)
    _check(case.replace("_long", "").replace("_pingpong", "").replace("_deep", "").replace("_rotated", ""), results, p2p)
    iterations = {"jacobi2d_long": 23, "jacobi3d_long": 9, "jacobi2d_pingpong": 11, "jacobi2d_deep": 70}
    for d in results:
        if case not in ("cg", "cg_rotated"):
            assert int(d["deep_halo_sweeps"]) > 0
            # one exchange serves `halo` sweeps (residual sweeps aside): fewer exchanges than sweeps
            assert int(d["halo_exchanges"]) < iterations[case]
