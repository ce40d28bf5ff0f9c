"""GPU tests of the launch-level options: programmatic dependent launches and the register cap
of the cache-served stencil kernels.  Neither may change a bit of any result: the same programs
run under every setting and are compared with the oracle each time."""
import os

import numpy as np
import pytest

import charmnumeric_b200 as cnp
from tests.helpers import run_both, assert_bit_exact, assert_rel

RTOL_REDUCTION = 1e-10  # dots and sums: tolerance of the north-star statement

pytestmark = pytest.mark.gpu


def _sweeps():
    """Many short kernels that each read what the previous one wrote."""
    u = cnp.random.uniform((130, 258), seed=301)
    u[0, :] = 1.0
    u[-1, :] = 0.0
    res = cnp.zeros((1,))
    for i in range(40):
        if i % 10 == 9:
            new = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:])
            d = new - u[1:-1, 1:-1]
            u[1:-1, 1:-1] = new
            res[...] = cnp.sum(d * d)
        else:
            u[1:-1, 1:-1] = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:])
    return {"u": u, "s_res": res}


def _wide_stencil():
    """A 9-point stencil over three arrays with two fused reductions: enough live values that
    a tight register cap cannot hold them."""
    a = cnp.random.uniform((67, 130), seed=311, low=-1.0, high=1.0)
    b = cnp.random.uniform((67, 130), seed=312, low=-1.0, high=1.0)
    c = cnp.random.uniform((67, 130), seed=313, low=-1.0, high=1.0)
    out = cnp.zeros((67, 130))
    out[1:-1, 1:-1] = (a[:-2, :-2] * b[1:-1, 1:-1] + a[:-2, 1:-1] * c[1:-1, 1:-1] + a[:-2, 2:] * b[2:, 2:]
                       + a[1:-1, :-2] * c[:-2, :-2] + 4.0 * a[1:-1, 1:-1] + a[1:-1, 2:] * b[:-2, 2:]
                       + a[2:, :-2] * c[2:, :-2] + a[2:, 1:-1] * b[2:, 1:-1] + a[2:, 2:] * c[1:-1, 2:]
                       - b[1:-1, :-2] * c[1:-1, 2:] - b[:-2, 1:-1] / (1.5 + c[2:, 1:-1] * c[2:, 1:-1]))
    return {"out": out, "s_oo": cnp.dot2d(out, out), "s_oa": cnp.dot2d(out, a)}


def _check(itf, prog):
    gpu, cpu = run_both(itf, prog)
    arrays = [k for k in cpu if not k.startswith("s_")]
    assert_bit_exact({k: gpu[k] for k in arrays}, {k: cpu[k] for k in arrays})
    scalars = {k: gpu[k] for k in cpu if k.startswith("s_")}
    assert_rel(scalars, {k: cpu[k] for k in scalars}, RTOL_REDUCTION)
    return gpu


def test_dependent_launch_on_and_off_agree(interface):
    ctx = interface.context
    try:
        ctx.set_option("dependent_launch", 0)
        off = _check(interface, _sweeps)
        ctx.set_option("dependent_launch", 1)
        on = _check(interface, _sweeps)
    finally:
        ctx.set_option("dependent_launch", 1)
    for k in off:
        assert off[k].tobytes() == on[k].tobytes(), k


@pytest.mark.parametrize("blocks", ["1", "6", "8"])
def test_register_cap_keeps_results(blocks, capfd):
    """Contexts compiled for 1 (no cap), 6 (default) and 8 resident blocks per SM.  The wide
    stencil needs about 84 registers: under a cap it would spill, so it must come out of the
    uncapped compile (more than 40 registers) whatever the setting; the 5-point sweep fits."""
    saved = {k: os.environ.get(k) for k in ("CN_STENCIL_BLOCKS", "CN_KERNEL_INFO")}
    os.environ["CN_STENCIL_BLOCKS"] = blocks
    os.environ["CN_KERNEL_INFO"] = "1"
    itf = None
    try:
        itf = cnp.CharmNumericInterface(device=int(os.environ.get("CN_TEST_DEVICE", "0")))
        _check(itf, _sweeps)
        _check(itf, _wide_stencil)
    finally:
        if itf is not None:
            itf.close()
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    info = [l for l in capfd.readouterr().err.splitlines() if l.startswith("[cnb200]")]
    regs = {}
    for line in info:   # "[cnb200] <entry> <label>: N registers, ..."
        entry = line.split()[1]
        regs[entry.rsplit("_", 1)[0]] = int(line.split(":")[-1].split("registers")[0])
    wide = [v for k, v in regs.items() if "shifted2d_i3o1" in k]
    sweep = [v for k, v in regs.items() if "shifted2d_i1o1r0" in k]
    assert wide and min(wide) > 40, regs
    if blocks != "1":
        assert sweep and max(sweep) <= 40, regs


def test_scalar_tail_on_and_off_agree(interface):
    """`res[...] = sum(d * d)` behind a sweep with a fused reduction: with the tail folded into
    the sweep's kernel and as a kernel of its own, the bits are the same and match the oracle."""
    ctx = interface.context
    try:
        ctx.set_option("fuse_scalar_tail", 0)
        before = ctx.stats()
        off = _check(interface, _sweeps)
        mid = ctx.stats()
        ctx.set_option("fuse_scalar_tail", 1)
        on = _check(interface, _sweeps)
        after = ctx.stats()
    finally:
        ctx.set_option("fuse_scalar_tail", 0)
    assert mid["scalar_tails"] == before["scalar_tails"]
    # inside one DAG the frontend puts size-1 arithmetic into the group that follows it; only
    # the last residual's `res[...] = s` stands alone behind its reduction
    tails = after["scalar_tails"] - mid["scalar_tails"]
    assert tails >= 1
    assert (after["kernel_launches"] - mid["kernel_launches"]) == (mid["kernel_launches"] - before["kernel_launches"]) - tails
    for k in off:
        assert off[k].tobytes() == on[k].tobytes(), k


def test_option_ranges(interface):
    """cn_set_option checks its values: halo depth 0..64, switches by name, nothing unknown."""
    from charmnumeric_b200._lib import CnError
    ctx = interface.context
    try:
        ctx.set_option("halo", 64)
        with pytest.raises(CnError):
            ctx.set_option("halo", 65)
        with pytest.raises(CnError):
            ctx.set_option("halo", -1)
        for key in ("dependent_launch", "fuse_scalar_tail"):
            ctx.set_option(key, 1)
            ctx.set_option(key, 0)
        with pytest.raises(CnError):
            ctx.set_option("no_such_option", 1)
    finally:
        ctx.set_option("halo", 1)
        ctx.set_option("dependent_launch", 1)
        ctx.set_option("fuse_scalar_tail", 0)
