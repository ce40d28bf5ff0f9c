"""Differential test of the lazy frontend (CPU only): seeded random programs -- elementwise
arithmetic on arrays, views and scalars, shifted and strided slices, in-place region updates
that read what they overwrite, reductions -- are executed eagerly with NumPy and lazily through
the frontend (grouping, temporaries, hazards, wire nodes) and the oracle interpreter; every
array must come out bit-identical.  A share of the programs also goes through the backend's
host-side compiler, so every group the frontend forms is one the DAG-group compiler accepts.

Only IEEE-exact operations are used (+, -, *, /, abs, sqrt): NumPy is then an exact oracle for
the oracle."""
import random

import numpy as np
import pytest

import charmnumeric_b200 as cnp
from tests.helpers import OracleInterface

SHAPES = [(13, 18), (41,), (6, 7, 10), (9, 32)]


def _random_view(rng, shape):
    """A pair of slices selecting a sub-box; the result extents are returned too."""
    sl, ext = [], []
    for n in shape:
        step = rng.choice([1, 1, 1, 2])
        lo = rng.randrange(0, 3)
        hi = n - rng.randrange(0, 3)
        sl.append(slice(lo, hi, step))
        ext.append(len(range(lo, hi, step)))
    return tuple(sl), tuple(ext)


def _same_extent_view(rng, shape, ext, step_ok=True):
    """Slices of the given extents, shifted at random (as the arms of a stencil are)."""
    sl = []
    for n, e in zip(shape, ext):
        step = rng.choice([1, 1, 2]) if step_ok else 1
        span = (e - 1) * step + 1
        if span > n:
            step, span = 1, e
        lo = rng.randrange(0, n - span + 1)
        sl.append(slice(lo, lo + span, step))
    return tuple(sl)


class _Pair:
    """The same value held eagerly (NumPy) and lazily (frontend)."""

    def __init__(self, eager, lazy):
        self.e, self.l = eager, lazy


def _operand(rng, arrays, ext, SHAPE, device_scalars=()):
    kind = rng.random()
    if kind < 0.2:
        v = rng.choice([2, -1, 3] if arrays[0].e.dtype.kind == "i" else [0.5, 2.0, -1.25, 3.0])
        return _Pair(v, v)
    if kind < 0.3 and device_scalars:
        # a size-1 device array (the alpha and beta of a CG iteration): broadcast like a scalar
        return rng.choice(device_scalars)
    a = rng.choice(arrays)
    sl = _same_extent_view(rng, SHAPE, ext)
    if rng.random() < 0.15:
        # the same elements through a view of a view (the outer view trims nothing or one
        # leading row, the inner slices are shifted accordingly)
        trim = 1 if sl[0].start >= 1 else 0
        outer = (slice(trim, None),) + (slice(None),) * (len(SHAPE) - 1)
        inner = (slice(sl[0].start - trim, sl[0].stop - trim, sl[0].step),) + tuple(sl[1:])
        return _Pair(a.e[outer][inner], a.l[outer][inner])
    return _Pair(a.e[sl], a.l[sl])


def _expression(rng, arrays, ext, depth, SHAPE, device_scalars=()):
    if depth == 0 or rng.random() < 0.25:
        x = _operand(rng, arrays, ext, SHAPE, device_scalars)
        if not isinstance(x.e, np.ndarray) or x.e.ndim == 0:  # keep at least one array in every expression
            y = _operand(rng, arrays, ext, SHAPE)
            while not isinstance(y.e, np.ndarray) or y.e.ndim == 0:
                y = _operand(rng, arrays, ext, SHAPE)
            return _Pair(x.e + y.e, x.l + y.l)
        return x
    integer = isinstance(arrays[0].e, np.ndarray) and arrays[0].e.dtype.kind == "i"
    op = rng.choice(["+", "-", "*", "abs", "neg"] if integer else ["+", "-", "*", "/", "abs", "sqrt", "neg"])
    a = _expression(rng, arrays, ext, depth - 1, SHAPE, device_scalars)
    if op == "abs":
        return _Pair(np.abs(a.e), cnp.abs(a.l))
    if op == "sqrt":
        return _Pair(np.sqrt(np.abs(a.e)), cnp.sqrt(cnp.abs(a.l)))
    if op == "neg":
        return _Pair(a.e * -1, -a.l)      # the reference's negation is a multiplication by -1
    b = _expression(rng, arrays, ext, depth - 1, SHAPE, device_scalars)
    if op == "+":
        return _Pair(a.e + b.e, a.l + b.l)
    if op == "-":
        return _Pair(a.e - b.e, a.l - b.l)
    if op == "*":
        return _Pair(a.e * b.e, a.l * b.l)
    # keep denominators away from zero so that no NaN / inf comparisons are needed
    return _Pair(a.e / (np.abs(b.e) + 1.0), a.l / (cnp.abs(b.l) + 1.0))


def _program(seed, interface, SHAPE=None):
    SHAPE = SHAPE or SHAPES[seed % len(SHAPES)]
    rng = random.Random(seed)
    nprng = np.random.default_rng(seed)
    arrays, scalars = [], []
    # some programs flush by themselves every few ops: results then live across batches
    if seed % 3 == 1:
        cnp.set_auto_flush(interface, rng.choice([2, 5, 11]))
    # every fifth program in single precision, every seventh on integers (no division, no sqrt)
    dtype = np.float32 if seed % 5 == 3 else (rng.choice([np.int32, np.int64]) if seed % 7 == 2 else np.float64)
    integer = np.dtype(dtype).kind == "i"
    for _ in range(3):
        host = (nprng.integers(-3, 4, SHAPE) if integer else nprng.uniform(-2.0, 2.0, SHAPE)).astype(dtype)
        arrays.append(_Pair(host.copy(), cnp.asarray(host)))
    # an array of exactly representable values: its sums and dot products are exact in any order,
    # so that scalars derived from them can flow back into array expressions bit for bit
    exact_host = nprng.choice(np.array([-1, 1, 2, 0] if integer else [-1.0, 0.5, 2.0, 0.25], dtype=dtype), SHAPE)
    exact = _Pair(exact_host.copy(), cnp.asarray(exact_host))
    device_scalars = []
    products = []       # results of non-fusible nodes (matvec), compared to 1e-10 at the end
    for _ in range(rng.randrange(4, 9)):
        if rng.random() < 0.25:
            if rng.random() < 0.5:
                device_scalars.append(_Pair(dtype(np.sum(exact.e)), cnp.sum(exact.l)))
            else:
                device_scalars.append(_Pair(dtype(np.sum(exact.e * exact.e)), cnp.dot2d(exact.l, exact.l)))
            if len(device_scalars) >= 2 and rng.random() < 0.5 and not integer:   # scalar-scalar arithmetic on the device
                a, b = device_scalars[-2], device_scalars[-1]
                device_scalars.append(_Pair(dtype(a.e / (abs(b.e) + dtype(1.0))), a.l / (cnp.abs(b.l) + 1.0)))
        if len(arrays) > 3 and rng.random() < 0.2:
            # drop an array: results nobody holds any more become temporaries of their group
            del arrays[rng.randrange(len(arrays))]
        if len(SHAPE) == 2 and rng.random() < 0.15 and not integer:
            # non-fusible nodes between the groups: a matvec with one of the arrays, and a tile
            # of a fresh vector that joins the arrays
            vec_host = nprng.uniform(-1.0, 1.0, (SHAPE[1],)).astype(dtype)
            vec = _Pair(vec_host, cnp.asarray(vec_host))
            a = rng.choice(arrays)
            products.append(_Pair(a.e.astype(np.float64) @ vec.e.astype(np.float64), a.l @ vec.l))
            arrays.append(_Pair(np.tile(vec.e, (SHAPE[0], 1)), cnp.tile(vec.l, (SHAPE[0], 1))))
        action = rng.random()
        if action < 0.55:                     # region update, possibly reading what it overwrites
            target = rng.choice(arrays)
            dst, ext = _random_view(rng, SHAPE)
            rhs = _expression(rng, arrays, ext, rng.randrange(1, 4), SHAPE, device_scalars)
            value = np.array(rhs.e, copy=True)   # the right-hand side is evaluated before the write
            target.e[dst] = value
            target.l[dst] = rhs.l
        elif action < 0.6 and len(SHAPE) >= 2:   # one row (plane) assigned from another through integer indices
            target, source = rng.choice(arrays), rng.choice(arrays)
            i, j = rng.randrange(SHAPE[0]), rng.randrange(SHAPE[0])
            value = np.array(source.e[j] * 2, copy=True)
            target.e[i] = value
            target.l[i] = source.l[j] * 2
        elif action < 0.75:                   # a new whole array from an expression
            rhs = _expression(rng, arrays, SHAPE, rng.randrange(1, 4), SHAPE, device_scalars)
            lazy = rhs.l.copy() if isinstance(rhs.l, cnp.ArrayView) else rhs.l   # a bare view aliases its base
            arrays.append(_Pair(np.array(rhs.e, copy=True), lazy))
        elif action < 0.9:                    # literal fill of a region
            target = rng.choice(arrays)
            dst, _ = _random_view(rng, SHAPE)
            v = rng.choice([0, 1, -3] if integer else [0.0, 1.0, -3.5])
            target.e[dst] = v
            target.l[dst] = v
        else:                                 # reduction of a fresh expression
            rhs = _expression(rng, arrays, SHAPE, 2, SHAPE)
            total = np.sum(rhs.e, dtype=np.int64).astype(dtype) if integer else np.sum(rhs.e)   # integer sums wrap
            scalars.append(_Pair(float(total), cnp.sum(rhs.l)))
    for a in arrays:
        got = a.l.get(interface)
        assert got.shape == a.e.shape
        assert got.tobytes() == np.ascontiguousarray(a.e).tobytes(), f"seed {seed}: array differs"
    for pr in products:
        got = np.asarray(pr.l.get(interface), np.float64)
        tol = 1e-10 if dtype == np.float64 else 1e-4
        assert np.max(np.abs(got - pr.e)) <= tol * max(1.0, float(np.max(np.abs(pr.e)))), f"seed {seed}: matvec differs"
    for s in scalars:
        got = float(s.l.get(interface)[0])
        tol = 1e-10 if dtype == np.float64 else 1e-4   # float32 sums: different summation orders
        assert abs(got - s.e) <= tol * max(1.0, abs(s.e)), f"seed {seed}: reduction differs"


@pytest.mark.parametrize("seed", range(80))
def test_random_programs_match_numpy(seed):
    cnp.reset_frontend_state()
    _program(seed, OracleInterface(dry_run=False))


@pytest.mark.parametrize("seed", range(1000, 1012))
def test_random_programs_lower_and_compile(seed):
    cnp.reset_frontend_state()
    itf = OracleInterface(dry_run=True)      # every fusible group goes through lower + NVRTC
    _program(seed, itf)
    assert itf.mirror.compiled > 0
