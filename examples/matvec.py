"""Matrix-vector product (the reference's examples/matvec.py, cross-partition form):
A[i, j] = i + j, x = 1.

    python examples/matvec.py [M]
"""
import sys

import numpy as np

import charmnumeric_b200 as cnp

M = int(sys.argv[1]) if len(sys.argv) > 1 else 48
interface = cnp.CharmNumericInterface(device=0)

A = cnp.zeros((M, M), dtype=cnp.float64)
for i in range(M):
    A[i, :] = float(i)
cols = cnp.zeros((M, M), dtype=cnp.float64)
for j in range(M):
    cols[:, j] = float(j)
A = A + cols
x = cnp.ones((M,), dtype=cnp.float64)
y = A.matvec(x)

result = y.get(interface)
expected = np.add.outer(np.arange(M, dtype=np.float64), np.arange(M, dtype=np.float64)) @ np.ones(M)
print("Match:", np.allclose(result, expected))
assert np.allclose(result, expected)
