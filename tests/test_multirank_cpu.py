"""CPU test of the multi-rank protocol: two gloo ranks run the slab-partitioned Jacobi sweep
with the same steps the GPU executor takes (slab range from cn_partition, one halo row per
side exchanged with the neighbours before the sweep, local sweep with the reference's
association order, residual = sum of the ranks' partial sums) and must reproduce the
single-process oracle bit for bit.  Only the arithmetic is numpy here; partition and
exchange pattern are the backend's."""
import ctypes as C
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n0, n1, iters, outdir):
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from charmnumeric_b200 import _lib
    from oracle import oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = _lib.load()
    b, e = C.c_int64(), C.c_int64()
    assert lib.cn_partition(n0, world, rank, C.byref(b), C.byref(e)) == 0
    rb, re = b.value, e.value
    nl = re - rb
    # local slab with one halo row on each side; seeded values by global index
    full = O.randu((n0, n1), 0x5EED + 1)
    full[0, :] = 1.0
    full[-1, :] = 0.0
    full[:, 0] = 0.0
    full[:, -1] = 0.0
    loc = np.zeros((nl + 2, n1))
    loc[1:-1] = full[rb:re]
    residuals = []
    for it in range(iters):
        # halo exchange: first row up, last row down (send/recv pairs, as the executor does)
        reqs = []
        up, down = rank - 1, rank + 1
        recv_top = torch.zeros(n1, dtype=torch.float64)
        recv_bot = torch.zeros(n1, dtype=torch.float64)
        if up >= 0 and nl > 0:
            reqs.append(dist.isend(torch.from_numpy(loc[1].copy()), up))
            reqs.append(dist.irecv(recv_top, up))
        if down < world and nl > 0:
            reqs.append(dist.isend(torch.from_numpy(loc[nl].copy()), down))
            reqs.append(dist.irecv(recv_bot, down))
        for r in reqs:
            r.wait()
        if up >= 0:
            loc[0] = recv_top.numpy()
        if down < world:
            loc[nl + 1] = recv_bot.numpy()
        # rows of the global interior [1, n0-1) that live here
        g_lo, g_hi = max(rb, 1), min(re, n0 - 1)
        new = loc.copy()
        part = 0.0
        if g_hi > g_lo:
            i0, i1 = g_lo - rb + 1, g_hi - rb + 1
            t = loc[i0 - 1:i1 - 1, 1:-1] + loc[i0 + 1:i1 + 1, 1:-1]
            t = t + loc[i0:i1, 0:-2]
            t = t + loc[i0:i1, 2:]
            v = 0.25 * t
            d = v - loc[i0:i1, 1:-1]
            part = float(O.dot(d, d, tile=1 << 30))
            new[i0:i1, 1:-1] = v
        loc = new
        tot = torch.tensor([part], dtype=torch.float64)
        dist.all_reduce(tot)
        residuals.append(float(tot[0]))
    np.save(os.path.join(outdir, f"slab{rank}.npy"), loc[1:-1])
    np.save(os.path.join(outdir, f"res{rank}.npy"), np.array(residuals))
    dist.destroy_process_group()


@pytest.mark.parametrize("n0,n1", [(16, 12), (11, 9)])
def test_two_rank_jacobi_matches_single_process_oracle(tmp_path, oracle_mod, n0, n1):
    import torch.multiprocessing as mp
    iters = 4
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n0, n1, iters, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = np.concatenate([np.load(tmp_path / f"slab{r}.npy") for r in range(2)], axis=0)
    res = np.load(tmp_path / "res0.npy")
    # single-process oracle: the C loops
    u = oracle_mod.randu((n0, n1), 0x5EED + 1)
    u[0, :] = 1.0
    u[-1, :] = 0.0
    u[:, 0] = 0.0
    u[:, -1] = 0.0
    scratch = np.zeros_like(u)
    want_res = np.zeros(iters)
    oracle_mod.clib().cno_jacobi2d(oracle_mod._ptr(u), oracle_mod._ptr(scratch), n0, n1, 0.25, iters, 1,
                                   oracle_mod._ptr(want_res), 1 << 20)
    assert got.tobytes() == u.tobytes()
    np.testing.assert_allclose(res, want_res, rtol=1e-12)
    assert np.array_equal(res, np.load(tmp_path / "res1.npy"))
