"""A DAG blob whose bytes have run before is served from the context's plan cache (parsing and
lowering skipped).  The results must not depend on it: every workload's step blobs give the same
bits with the cache on and off, the array table is still consulted per run, and changing an
option that lowering looks at drops the cached plans."""
import numpy as np
import pytest

import charmnumeric_b200 as cnp
from charmnumeric_b200 import _lib
from charmnumeric_b200.workloads import CG, Jacobi2D, Jacobi3D

pytestmark = pytest.mark.gpu


def _run_steps(interface, make, steps, cache):
    cnp.reset_frontend_state()
    ctx = interface.context
    ctx.set_option("plan_cache", cache)
    w = make(interface)
    before = ctx.stats()["plan_hits"]
    scalars = []
    for i in range(steps):
        w.run_step(i)
        scalars.append(w.read_result())
    hits = ctx.stats()["plan_hits"] - before
    fields = {a.name: ctx.get(a.name) for a in w.keep if a.size > 1}
    return scalars, fields, hits


@pytest.mark.parametrize("make,steps", [
    (lambda itf: Jacobi2D(itf, scale=0.07, res_every=3), 12),
    (lambda itf: Jacobi3D(itf, scale=0.04, res_every=2), 6),
    (lambda itf: CG(itf, scale=0.02), 8),
], ids=["jacobi2d", "jacobi3d", "cg"])
def test_cached_plans_give_the_same_bits(interface, make, steps):
    try:
        s_off, f_off, hits_off = _run_steps(interface, make, steps, 0)
        s_on, f_on, hits_on = _run_steps(interface, make, steps, 1)
    finally:
        interface.context.set_option("plan_cache", 1)
    assert hits_off == 0
    assert hits_on >= steps - 2          # every blob misses once, then hits
    assert np.array(s_on).tobytes() == np.array(s_off).tobytes()
    assert len(f_on) == len(f_off) > 0
    for a, b in zip(f_on.values(), f_off.values()):
        assert a.tobytes() == b.tobytes()


def test_cached_plan_still_checks_the_array_table(interface):
    ctx = interface.context
    w = Jacobi2D(interface, scale=0.05, res_every=0)
    w.run_step(0)
    w.run_step(1)                        # served from the cache
    ctx.synchronize()
    ctx.delete_array(w.u.name)
    with pytest.raises(_lib.CnError) as e:
        w.run_step(2)
    assert e.value.status == 3       # CN_STATUS_UNKNOWN_ARRAY


def test_option_change_drops_cached_plans(interface):
    ctx = interface.context
    w = Jacobi3D(interface, scale=0.04, res_every=0)
    try:
        w.run_step(0)
        w.run_step(1)
        staged0 = ctx.stats()["group_launches"]
        h0 = ctx.stats()["plan_hits"]
        ctx.set_option("staged", 0)      # the next run must lower again, to the cache-served kernel
        w.run_step(2)
        assert ctx.stats()["plan_hits"] == h0
        w.run_step(3)
        assert ctx.stats()["plan_hits"] == h0 + 1
        assert ctx.stats()["group_launches"] >= staged0 + 2
    finally:
        ctx.set_option("staged", 1)
    ctx.synchronize()
