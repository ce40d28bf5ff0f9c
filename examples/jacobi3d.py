"""3-D Jacobi iteration (the reference's examples/jacobi3d.py) with a residual every 10 sweeps.

    python examples/jacobi3d.py [n] [iterations]
"""
import sys

import charmnumeric_b200 as cnp

n = int(sys.argv[1]) if len(sys.argv) > 1 else 128
iters = int(sys.argv[2]) if len(sys.argv) > 2 else 100

interface = cnp.CharmNumericInterface(device=0)
u = cnp.zeros((n, n, n), dtype=cnp.float64)
u[0, :, :] = 1.0
u[-1, :, :] = 1.0
u[:, 0, :] = 1.0
u[:, -1, :] = 1.0
u[:, :, 0] = 1.0
u[:, :, -1] = 1.0

c = 0.16666666666666666
for it in range(1, iters + 1):
    new = c * (u[:-2, 1:-1, 1:-1] + u[2:, 1:-1, 1:-1] + u[1:-1, :-2, 1:-1]
               + u[1:-1, 2:, 1:-1] + u[1:-1, 1:-1, :-2] + u[1:-1, 1:-1, 2:])
    if it % 10 == 0:
        d = new - u[1:-1, 1:-1, 1:-1]
        sq = d * d
        u[1:-1, 1:-1, 1:-1] = new
        res = cnp.sum(sq)          # fused into the sweep's kernel
        del d, sq
        print(f"iteration {it}: sum((new-old)^2) = {res.get(interface).item():.6e}")
    else:
        u[1:-1, 1:-1, 1:-1] = new
    del new

print(u.get(interface)[n // 2, n // 2, :8])
