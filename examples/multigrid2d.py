"""Geometric multigrid V-cycles for -laplacian(u) = f on the unit square with zero Dirichlet
boundary (the solver of the reference's examples/multigrid2d.py, on the B200 backend):
weighted-Jacobi smoothing, 9-point full-weighting restriction, bilinear prolongation.

Every operator is written once against the array API that both NumPy arrays and backend arrays
offer, so the same functions build the backend's DAGs and compute the NumPy answer the result is
compared with.

    python examples/multigrid2d.py [n = 2^k + 1] [cycles]
"""
import sys

import numpy as np

import charmnumeric_b200 as cnp

OMEGA = 2.0 / 3.0


def smooth(u, f, h2, sweeps):
    for _ in range(sweeps):
        jac = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:] + h2 * f[1:-1, 1:-1])
        u[1:-1, 1:-1] = (1.0 - OMEGA) * u[1:-1, 1:-1] + OMEGA * jac


def residual(u, f, h2, zeros):
    r = zeros(u.shape)
    r[1:-1, 1:-1] = f[1:-1, 1:-1] - (1.0 / h2) * (
        4.0 * u[1:-1, 1:-1] - u[:-2, 1:-1] - u[2:, 1:-1] - u[1:-1, :-2] - u[1:-1, 2:])
    return r


def restrict(fine, zeros):
    nc = (fine.shape[0] - 1) // 2 + 1
    coarse = zeros((nc, nc))
    c, lo, hi = slice(2, -2, 2), slice(1, -3, 2), slice(3, -1, 2)
    coarse[1:-1, 1:-1] = (
        0.25 * fine[c, c]
        + 0.125 * (fine[lo, c] + fine[hi, c] + fine[c, lo] + fine[c, hi])
        + 0.0625 * (fine[lo, lo] + fine[lo, hi] + fine[hi, lo] + fine[hi, hi]))
    return coarse


def prolongate_add(e, u, zeros):
    fine = zeros(u.shape)
    fine[2:-2:2, 2:-2:2] = e[1:-1, 1:-1]
    fine[1:-1:2, 2:-2:2] = 0.5 * (e[:-1, 1:-1] + e[1:, 1:-1])
    fine[2:-2:2, 1:-1:2] = 0.5 * (e[1:-1, :-1] + e[1:-1, 1:])
    fine[1:-1:2, 1:-1:2] = 0.25 * (e[:-1, :-1] + e[1:, :-1] + e[:-1, 1:] + e[1:, 1:])
    u[1:-1, 1:-1] = u[1:-1, 1:-1] + fine[1:-1, 1:-1]


def vcycle(u, f, h, zeros, pre=2, post=2, coarse_sweeps=50):
    h2 = h * h
    if u.shape[0] <= 5:
        smooth(u, f, h2, coarse_sweeps)
        return
    smooth(u, f, h2, pre)
    rc = restrict(residual(u, f, h2, zeros), zeros)
    ec = zeros(rc.shape)
    vcycle(ec, rc, 2.0 * h, zeros, pre, post, coarse_sweeps)
    prolongate_add(ec, u, zeros)
    smooth(u, f, h2, post)


def main():
    n = int(sys.argv[1]) if len(sys.argv) > 1 else 129
    cycles = int(sys.argv[2]) if len(sys.argv) > 2 else 3
    if (n - 1) & (n - 2) or n < 5:
        raise SystemExit("n must be 2^k + 1")
    h = 1.0 / (n - 1)
    xs = np.linspace(0.0, 1.0, n)
    f_host = 2.0 * np.pi ** 2 * np.outer(np.sin(np.pi * xs), np.sin(np.pi * xs))
    exact = np.outer(np.sin(np.pi * xs), np.sin(np.pi * xs))

    interface = cnp.CharmNumericInterface(device=0)
    cnp.set_auto_flush(interface, 100000)
    f = cnp.array(f_host)
    u = cnp.zeros((n, n), dtype=cnp.float64)
    for _ in range(cycles):
        vcycle(u, f, h, lambda s: cnp.zeros(tuple(s), dtype=cnp.float64))
    got = u.get(interface)

    u_np = np.zeros((n, n))
    for _ in range(cycles):
        vcycle(u_np, f_host, h, lambda s: np.zeros(tuple(s)))

    err = np.max(np.abs(got - exact))
    print(f"multigrid n={n}, {cycles} V-cycles: max |u - exact| = {err:.3e}")
    ok = np.array_equal(got, u_np)
    print("bit-exact with NumPy:", ok)
    sys.exit(0 if ok else 1)


main()
