"""Jacobi iteration x <- x + D^-1 (b - A x) for a diagonally dominant dense system (the program
of the reference's examples/jacobi_iteration.py, on the B200 backend): diag builds the matrix
and extracts its diagonal, each iteration is one matvec and one fused elementwise group.

    python examples/jacobi_iteration.py [n] [iterations]
"""
import sys

import numpy as np

import charmnumeric_b200 as cnp

n = int(sys.argv[1]) if len(sys.argv) > 1 else 128
iters = int(sys.argv[2]) if len(sys.argv) > 2 else 50

interface = cnp.CharmNumericInterface(device=0)

# A = ones + 2n I: symmetric, strictly diagonally dominant
A = cnp.ones((n, n), dtype=cnp.float64) + cnp.diag(cnp.full((n,), 2.0 * n, dtype=cnp.float64))
b = cnp.ones((n,), dtype=cnp.float64)
d = cnp.diag(A)
d_host = d.get(interface)
assert np.array_equal(d_host, np.full(n, 2.0 * n + 1.0)), "diag(A) came back wrong"
d_inv = 1.0 / d

x = cnp.zeros((n,), dtype=cnp.float64)
for _ in range(iters):
    x = x + d_inv * (b - A @ x)
result = x.get(interface)

A_np = np.ones((n, n)) + 2.0 * n * np.eye(n)
x_np = np.linalg.solve(A_np, np.ones(n))
err = np.max(np.abs(result - x_np))
print(f"Jacobi iteration ({iters} iterations, n={n}): max error vs numpy.linalg.solve = {err:.2e}")
ok = bool(np.allclose(result, x_np, atol=1e-6))
print("converged:", ok)
sys.exit(0 if ok else 1)
