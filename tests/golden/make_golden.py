"""Regenerate the committed golden fixtures.

The reference ships no golden files and cannot be imported or built in this environment
(charmtyles, Charm++, MLIR and Eigen are absent), so the fixtures hold what the reference's
own tests compare against -- the NumPy value of each test expression
(tests/test_backend_integration.py:13-127, examples/cg.py:65-73, examples/matvec.py:45-55) --
plus known answers of the seeded generator computed by an independent pure-Python
implementation.  Run:  python tests/golden/make_golden.py
"""
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
MASK = (1 << 64) - 1


def splitmix_unit(seed, g):
    z = (seed + (g + 1) * 0x9E3779B97F4A7C15) & MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    z = z ^ (z >> 31)
    return (z >> 11) * 2.0 ** -53


def main():
    vals = [0.0 + (1.0 - 0.0) * splitmix_unit(0x5EED, g) for g in range(4)]
    (HERE / "randu_5eed.txt").write_text("\n".join(v.hex() for v in vals) + "\n")

    kats = {}
    kats["expr_f32"] = np.full((32,), 8.0, dtype=np.float32)
    host = np.arange(512, dtype=np.float32)
    kats["shifted_f32"] = host[100:300] + host[150:350]
    n = 17
    cn = (n - 1) // 2 + 1
    want = np.zeros((cn, cn))
    want[1:-1, 1:-1] = np.ones((n, n))[2:-2:2, 2:-2:2]
    kats["strided_f64"] = want
    w = np.zeros((4, 4, 4), dtype=np.float32)
    w[0] = 1; w[-1] = 1; w[:, 0] = 1; w[:, -1] = 1; w[:, :, 0] = 1; w[:, :, -1] = 1
    w[1:-1, 1:-1, 1:-1] = (1.0 / 6.0) * (w[:-2, 1:-1, 1:-1] + w[2:, 1:-1, 1:-1] + w[1:-1, :-2, 1:-1]
                                         + w[1:-1, 2:, 1:-1] + w[1:-1, 1:-1, :-2] + w[1:-1, 1:-1, 2:])
    kats["jacobi3d_f32"] = w
    N = 128
    A = np.ones((N, N)) + N * np.eye(N)
    b = np.arange(1, N + 1, dtype=np.float64)
    kats["cg_solution"] = np.linalg.solve(A, b)
    M = 48
    kats["matvec_ipj"] = np.add.outer(np.arange(M, dtype=np.float64), np.arange(M, dtype=np.float64)) @ np.ones(M)
    for k in (0, 1, -1):  # tests/test_backend_integration.py:108-116
        kats[f"diag_vector_k{k}"] = np.diag(np.full(8, 2.0), k=k)
    kats["diag_matrix_k2"] = np.diag(np.full((6, 10), 3.0), k=2)  # :119-127
    np.savez(HERE / "reference_kats.npz", **kats)


if __name__ == "__main__":
    main()
