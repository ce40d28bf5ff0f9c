"""Worker of the multi-GPU tests: one process per GPU.  Usage:
    python tests/multi_worker.py <rank> <nranks> <id-file> <out-dir> <case>
Rank 0 writes the 128-byte communicator id to <id-file>; the others wait for it."""
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

import charmnumeric_b200 as cnp  # noqa: E402
from charmnumeric_b200 import frontend as F  # noqa: E402
from oracle.oracle import Oracle  # noqa: E402
from tests import test_gpu_parity as G  # noqa: E402


def main():
    rank, nranks, idfile, outdir, case = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5]
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if rank == 0:
        uid = cnp.comm_unique_id()
        tmp = idfile + ".tmp"
        Path(tmp).write_bytes(uid)
        os.replace(tmp, idfile)
    else:
        t0 = time.time()
        while not os.path.exists(idfile):
            if time.time() - t0 > 120:
                raise SystemExit("timed out waiting for the communicator id")
            time.sleep(0.05)
        uid = Path(idfile).read_bytes()
    itf = cnp.CharmNumericInterface(device=rank, rank=rank, nranks=nranks, unique_id=uid)
    progs = {
        "jacobi2d": G._jacobi2d_program(67, 130, 6, res_every=3),
        "jacobi2d_small": G._jacobi2d_program(9, 8, 3),
        "jacobi2d_long": G._jacobi2d_program(67, 130, 23, res_every=5),
        "jacobi2d_deep": G._jacobi2d_program(300, 130, 70, res_every=10),
        "jacobi3d_long": G._jacobi3d_program((26, 12, 34), 9),
        "jacobi3d": G._jacobi3d_program((19, 12, 34), 3),
        "cg": G._cg_poisson_program(34, 8),
    }

    def chain():
        a = cnp.random.uniform((100003,), seed=2, low=-1.0, high=1.0)
        b = cnp.random.uniform((100003,), seed=3, low=-1.0, high=1.0)
        return {"r": G._chain(a, b), "s": cnp.sum(G._chain(a, b)), "d": cnp.dot2d(a, b)}

    def matvec():
        A = cnp.random.uniform((301, 128), seed=21, low=-1.0, high=1.0)
        x = cnp.random.uniform((128,), seed=22, low=-1.0, high=1.0)
        y = A @ x
        # a row / column slice: the rows of A behind a rank's rows of the result live on other ranks
        ys = A[30:250, 16:100].matvec(x[16:100])
        return {"y": y, "n": y @ y, "ys": ys}

    def diag():
        n = 75
        A = cnp.random.uniform((n, n), seed=31, low=-1.0, high=1.0) + cnp.diag(cnp.full((n,), 2.0 * n))
        d = cnp.diag(A)
        x = cnp.random.uniform((n,), seed=32)
        tall = cnp.random.uniform((90, 40), seed=33)
        return {"A": A, "d": d, "x1": x + (1.0 / d) * (cnp.ones((n,)) - A @ x),
                # diagonals off the main one, and of a tall matrix: the rows behind a rank's part
                # of the result live on other ranks
                "up": cnp.diag(x, 2), "down": cnp.diag(x, -5), "d_up": cnp.diag(A, 3), "d_down": cnp.diag(A, -7),
                "d_tall": cnp.diag(tall), "d_tall_down": cnp.diag(tall, -30)}

    def tile():
        h0 = cnp.random.uniform((37,), seed=41)
        m = cnp.random.uniform((5, 6), seed=42)
        return {"rows": cnp.tile(h0, (11, 1)), "blocks": cnp.tile(m, (3, 2)), "cube": cnp.tile(h0, (2, 3, 1))}
    def pingpong():
        # two arrays written in turn, side boundaries that are not zero: a sweep writes the
        # interior region only, so the halo cells of the side columns keep what they held
        n0, n1 = 67, 130
        x = cnp.random.uniform((n0, n1), seed=51)
        xn = cnp.zeros((n0, n1))
        for u in (x, xn):
            u[0, :] = 1.0
            u[-1, :] = 0.5
            u[:, 0] = 1.0
            u[:, -1] = 2.0
        for it in range(11):
            xn[1:-1, 1:-1] = 0.25 * (x[:-2, 1:-1] + x[2:, 1:-1] + x[1:-1, :-2] + x[1:-1, 2:])
            x, xn = xn, x
        return {"x": x, "xn": xn}
    progs["jacobi2d_pingpong"] = pingpong
    import __graft_entry__ as entry_points
    progs["multigrid"] = entry_points._multigrid(65, 91)
    progs["cg_rotated"] = entry_points._cg_rotated(70, 34, 9)
    progs["xset"] = G._cross_dimension_program
    progs["chain"] = chain
    progs["diag"] = diag
    progs["tile"] = tile
    progs["matvec"] = matvec
    cnp.reset_frontend_state()
    outs = progs[case]()
    orc = Oracle()
    F.execute(itf, mirror=orc)
    result = {}
    for k, v in outs.items():
        result["gpu_" + k] = itf.context.get(v.name).reshape(v.shape)
        result["cpu_" + k] = np.array(orc.get(v.name)).reshape(v.shape)
    if case == "matvec":
        # the root-only gather: rank 1 receives the array, every other rank gets nothing
        y = outs["y"]
        rooted = itf.context.get_root(y.name, root=1)
        assert (rooted is not None) == (rank == 1)
        if rank == 1:
            assert rooted.tobytes() == result["gpu_y"].tobytes()
        # slab-wise upload: every rank hands in only its own rows
        rng = np.random.default_rng(5)
        whole = rng.uniform(-1.0, 1.0, (301, 7))
        b, e = cnp.partition(301, nranks, rank)
        itf.context.put_local(999001, whole.shape, whole[b:e])
        assert itf.context.get(999001).tobytes() == whole.tobytes()
    st = itf.context.stats()
    result["halo_exchanges"] = np.array(st["halo_exchanges"])
    result["allreduces"] = np.array(st["allreduces"])
    result["peer_exchanges"] = np.array(st["peer_exchanges"])
    result["overlapped_sweeps"] = np.array(st["overlapped_sweeps"])
    result["deep_halo_sweeps"] = np.array(st["deep_halo_sweeps"])
    result["row_fetches"] = np.array(st["row_fetches"])
    result["halo_pushes"] = np.array(st["halo_pushes"])
    result["inlined_producers"] = np.array(st["inlined_producers"])
    np.savez(os.path.join(outdir, f"{case}_rank{rank}.npz"), **result)
    itf.close()


if __name__ == "__main__":
    main()
