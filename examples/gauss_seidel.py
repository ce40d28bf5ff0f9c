"""Red-black Gauss-Seidel for -laplacian(phi) = f on the unit square, zero Dirichlet boundary
(the program of the reference's examples/gauss_seidel.py, on the B200 backend).  The four
colour/parity classes are strided views; each sweep is four strided DAG groups.  The result is
checked against the same sweeps done with NumPy.

    python examples/gauss_seidel.py [n] [iterations]
"""
import sys

import numpy as np

import charmnumeric_b200 as cnp

n = int(sys.argv[1]) if len(sys.argv) > 1 else 512
iters = int(sys.argv[2]) if len(sys.argv) > 2 else 10
h2 = (1.0 / (n - 1)) ** 2

# (rows, cols) start offsets of the four classes: red = (odd, odd), (even, even);
# black = (odd, even), (even, odd)
CLASSES = [(1, 1), (2, 2), (1, 2), (2, 1)]


def sweep(phi, f):
    for r0, c0 in CLASSES:
        rows, cols = slice(r0, -1, 2), slice(c0, -1, 2)
        up, down = slice(r0 - 1, -2, 2), slice(r0 + 1, None, 2)
        left, right = slice(c0 - 1, -2, 2), slice(c0 + 1, None, 2)
        phi[rows, cols] = 0.25 * (phi[up, cols] + phi[down, cols] + phi[rows, left] + phi[rows, right]
                                  - h2 * f[rows, cols])


interface = cnp.CharmNumericInterface(device=0)

phi = cnp.zeros((n, n), dtype=cnp.float64)
f = cnp.zeros((n, n), dtype=cnp.float64)
f[n // 2, n // 2] = -100.0
for _ in range(iters):
    sweep(phi, f)
result = phi.get(interface)

phi_np = np.zeros((n, n))
f_np = np.zeros((n, n))
f_np[n // 2, n // 2] = -100.0
for _ in range(iters):
    sweep(phi_np, f_np)

print(f"Gauss-Seidel ({iters} iterations, n={n}): phi max {result.max():.6e}, min {result.min():.6e}")
ok = np.array_equal(result, phi_np)
print("bit-exact with NumPy:", ok)
sys.exit(0 if ok else 1)
