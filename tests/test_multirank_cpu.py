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


def _restrict_worker(rank, world, port, n, outdir):
    """Full-weighting-style restriction coarse[1:-1] = 0.5 fine[2:-2:2] + 0.25 (fine[1:-3:2] +
    fine[3:-1:2]) on slabs: the rows a rank reads but does not own travel as the library's
    transfer plan says, then every rank computes its own iteration rows."""
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from charmnumeric_b200 import _lib
    from oracle import oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = _lib.load()
    nc = (n - 1) // 2 + 1
    fine = O.randu((n, 7), 77)

    def own(n0, q):
        b, e = C.c_int64(), C.c_int64()
        assert lib.cn_partition(n0, world, q, C.byref(b), C.byref(e)) == 0
        return b.value, e.value
    fb, fe = own(n, rank)
    cb, ce = own(nc, rank)
    mine = fine[fb:fe].copy()               # this rank holds only its slab of the fine grid
    anchor = (C.c_int64 * 3)(1, nc - 1, 1)  # coarse[1:-1]
    views = {"c": (2, n - 2, 2), "lo": (1, n - 3, 2), "hi": (3, n - 1, 2)}
    fetched = {}
    for key, view in views.items():
        leaf = (C.c_int64 * 3)(*view)
        count = C.c_int64()
        buf = (C.c_int64 * (4 * world * world + 4))()
        rows = (C.c_int64 * (2 * world))()
        assert lib.cn_plan_row_transfers(anchor, nc, leaf, n, world, buf, world * world + 1, C.byref(count), rows) == 0
        i0, i1 = rows[2 * rank], rows[2 * rank + 1]
        lo = view[0] + i0 * view[2] if i1 > i0 else 0
        hi = view[0] + (i1 - 1) * view[2] + 1 if i1 > i0 else 0
        scratch = np.full((max(hi - lo, 0), 7), np.nan)
        o0, o1 = max(lo, fb), min(hi, fe)
        if o1 > o0:
            scratch[o0 - lo:o1 - lo] = mine[o0 - fb:o1 - fb]
        reqs, landing = [], []
        for k in range(count.value):
            src, dst, t0, t1 = buf[4 * k:4 * k + 4]
            if src == rank:
                reqs.append(dist.isend(torch.from_numpy(mine[t0 - fb:t1 - fb].copy()), dst))
            if dst == rank:
                t = torch.zeros((t1 - t0, 7), dtype=torch.float64)
                reqs.append(dist.irecv(t, src))
                landing.append((t0, t1, t))
        for r in reqs:
            r.wait()
        for t0, t1, t in landing:
            scratch[t0 - lo:t1 - lo] = t.numpy()
        fetched[key] = (lo, scratch, i0, i1)
    lo_c, sc, i0, i1 = fetched["c"]
    out = np.zeros((ce - cb, 7))
    if i1 > i0:
        def rows_of(key):
            lo, scratch, a0, a1 = fetched[key]
            idx = views[key][0] + np.arange(a0, a1) * views[key][2] - lo
            return scratch[idx]
        val = 0.5 * rows_of("c") + 0.25 * (rows_of("lo") + rows_of("hi"))
        assert not np.isnan(val).any()
        first = 1 + i0 - cb                  # coarse row of iteration row i0, local
        out[first:first + (i1 - i0)] = val
    np.save(os.path.join(outdir, f"coarse{rank}.npy"), out)
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 33), (3, 65), (4, 17)])
def test_stepped_views_across_slabs_follow_the_transfer_plan(tmp_path, oracle_mod, world, n):
    import torch.multiprocessing as mp
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_restrict_worker, args=(r, world, port, n, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = np.concatenate([np.load(tmp_path / f"coarse{r}.npy") for r in range(world)], axis=0)
    fine = oracle_mod.randu((n, 7), 77)
    want = np.zeros(((n - 1) // 2 + 1, 7))
    want[1:-1] = 0.5 * fine[2:-2:2] + 0.25 * (fine[1:-3:2] + fine[3:-1:2])
    assert got.tobytes() == want.tobytes()
