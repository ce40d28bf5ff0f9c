"""2-D Jacobi iteration (the reference's examples/jacobi2d.py, float64, on the B200 backend).

    python examples/jacobi2d.py [n] [iterations]
"""
import sys

import charmnumeric_b200 as cnp

n = int(sys.argv[1]) if len(sys.argv) > 1 else 2048
iters = int(sys.argv[2]) if len(sys.argv) > 2 else 100

interface = cnp.CharmNumericInterface(device=0)
cnp.set_auto_flush(interface, 1000)

u = cnp.zeros((n, n), dtype=cnp.float64)
u[0, :] = 1.0
u[-1, :] = 1.0
u[:, 0] = 1.0
u[:, -1] = 1.0

for it in range(iters):
    u[1:-1, 1:-1] = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:])

print(u.get(interface))
