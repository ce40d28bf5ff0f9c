"""Conjugate gradient on a dense SPD system (the reference's examples/cg.py): A = ones + N*I,
b = 1..N, checked against numpy.linalg.solve.

    python examples/cg.py [N] [iterations]
"""
import sys

import numpy as np

import charmnumeric_b200 as cnp

N = int(sys.argv[1]) if len(sys.argv) > 1 else 128
max_iter = int(sys.argv[2]) if len(sys.argv) > 2 else 4

interface = cnp.CharmNumericInterface(device=0)
A_np = np.ones((N, N)) + N * np.eye(N)
A = cnp.asarray(A_np)
b = cnp.arange(1, N + 1, dtype=cnp.float64)

x = cnp.zeros((N,), dtype=cnp.float64)
r = b.copy()
p = b.copy()
rtr = r @ r

for k in range(max_iter):
    Ap = A @ p
    pAp = p @ Ap
    alpha = rtr / pAp
    x = x + alpha * p
    r = r - alpha * Ap
    rtr_new = r @ r
    beta = rtr_new / rtr
    p = r + beta * p
    rtr = rtr_new
    print(f"  iter {k + 1}: rtr = {rtr.get(interface).item():.6e}")

result = x.get(interface)
expected = np.linalg.solve(A_np, np.arange(1, N + 1, dtype=np.float64))
print("Match:", np.allclose(result, expected))
assert np.allclose(result, expected)
