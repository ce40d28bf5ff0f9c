"""The five benchmark workloads, written against the public lazy-array API.

Each workload records its set-up with the frontend, executes it, then records ONE steady-state
step in in-place form (every array keeps its name from step to step) and serialises it to a
DAG blob.  Re-submitting that blob through ``cn_receive_dag`` is one step; nothing but the
blob crosses the host/device boundary per step.

Shapes follow the five configurations the backend is measured on:
  jacobi2d  5-point Jacobi, 2048 x 2048 float64, residual sum((new-old)^2) every 10th step
  chain     s = sum(exp(-a*a)*b + sqrt(abs(a)) - 0.5*b*b + a/(1+abs(b))), n = 2^28
  cg        matrix-free CG, 2-D Poisson 5-point, 8192 x 8192 unknowns (zero Dirichlet ring)
  matvec    power iteration y = A x; x = y / sqrt(y.y), A 65536 x 65536 (32 GiB)
  jacobi3d  7-point Jacobi, 1024^3 float64
Inputs are synthetic: seeded uniform values generated on the device.
"""
from . import frontend as F
from . import wire

SEED = 0x5EED


def _capture_step(record):
    """Record one step with the frontend and return its nodes (nothing is executed)."""
    saved, F._state.pending = F._state.pending, []
    try:
        record()
        items = F.build_nodes(F._state.pending)
    finally:
        F._state.pending = saved
    nodes = []
    for kind, item in items:
        if kind != "node":
            raise RuntimeError("a benchmark step must not upload host data")
        nodes.append(item)
    return nodes


class Workload:
    name = ""
    metric = ""
    unit = "iterations/s"
    scaling = "weak"

    def __init__(self, interface, nranks=1, scale=1.0):
        self.itf = interface
        self.ctx = interface.context
        self.nranks = nranks
        self.scale = scale
        self.keep = []          # lazy arrays that must stay alive
        self.blobs = []         # step blobs; step i uses blobs[self.pick(i)]
        self.nodes = []         # the node lists behind the blobs (for the oracle in tests)
        self.result = None      # size-1 array read back per step in the end-to-end leg
        d = self.describe(nranks, scale)
        self.shape = d["shape"]
        self.points = d["points"]                  # grid points / elements / matrix entries per step (all ranks)
        self.bytes_per_step = d["bytes_per_step"]  # algorithmic HBM bytes per step, all ranks
        self.description = d["description"]
        self._result_host = None
        self._align_src = F.zeros((8,))  # created by the subclass's first execute
        self._align_blob = None

    def align_blob(self):
        """A DAG whose only work is a sum over a tiny array: on several ranks that is one
        allreduce, i.e. a barrier on the devices.  Submitted right before a timed burst it lines
        the ranks' streams up, so that the burst does not start with one GPU waiting for the
        others to be given their work."""
        if self._align_blob is None:
            def record():
                self.keep.append(F.sum_all(self._align_src))
            self._align_blob = wire.dag_blob(_capture_step(record))
        return self._align_blob

    @classmethod
    def describe(cls, nranks=1, scale=1.0):
        """Shape, size and description of the workload; needs no GPU (the CPU arm of the
        benchmark reports the same configuration string)."""
        raise NotImplementedError

    def release(self):
        """Drop every array of the workload and let the backend free them."""
        import gc
        self.keep = []
        self.result = None
        for key, value in list(vars(self).items()):
            if isinstance(value, (F.Array, F.ArrayView)):
                setattr(self, key, None)
        gc.collect()
        F.execute(self.itf)

    def pick(self, step_index):
        return 0

    def add_step(self, record):
        nodes = _capture_step(record)
        self.nodes.append(nodes)
        self.blobs.append(wire.dag_blob(nodes))

    def run_step(self, i):
        self.ctx.receive_dag(self.blobs[self.pick(i)])

    def read_result(self):
        """The step's size-1 result, read back into a host buffer that is allocated once."""
        if self._result_host is None:
            import numpy as np
            self._result_host = np.zeros((1,), dtype=np.float64)
        self.ctx.get_into(self.result.name, self._result_host)
        return float(self._result_host[0])


class CG(Workload):
    """examples/cg.py:26-52 with a matrix-free operator; two array kernels per step:
    (p update, Ap, p.Ap) | (x, r updates, r.r), and one size-1 kernel (beta, rtr carry)."""
    name = "cg"
    metric = "cg_iterations_per_sec"

    @classmethod
    def describe(cls, nranks=1, scale=1.0):
        n = max(8, int(8192 * scale))
        m0, m1 = n * nranks + 2, n + 2
        return {"shape": (m0, m1), "points": (m0 - 2) * (m1 - 2), "bytes_per_step": 80 * n * n * nranks,
                "description": (f"C3 matrix-free CG, 2-D Poisson 5-point, {n}x{n} unknowns per GPU "
                                f"(global {m0 - 2}x{m1 - 2}), one stencil matvec + two dots + three "
                                "axpys per iteration, slab decomposition")}

    def __init__(self, interface, nranks=1, scale=1.0):
        super().__init__(interface, nranks, scale)
        b = F.zeros(self.shape)
        b[1:-1, 1:-1] = F.uniform(self.shape, seed=SEED + 3)[1:-1, 1:-1]
        x = F.zeros(self.shape)
        r = b.copy()
        p = b.copy()
        Ap = F.zeros(self.shape)
        rtr = F.dot2d(r, r)
        beta = F.zeros((1,))
        F.execute(interface)
        self.keep = [b, x, r, p, Ap, rtr, beta]
        self.b, self.x, self.r, self.p, self.Ap, self.rtr, self.beta = b, x, r, p, Ap, rtr, beta
        self.result = rtr

        # One iteration of examples/cg.py:38-52, entered at the update of the search direction:
        # p = r + beta p (beta = 0 before the first iteration, so p = r), Ap, alpha, x, r,
        # beta.  The same operations on the same values as the loop written from `Ap = A p`
        # on; in this order the direction update sits right in front of the stencil that reads
        # it, and the backend runs the two as one kernel.
        def step():
            p[...] = r + beta * p
            Ap[1:-1, 1:-1] = (4.0 * p[1:-1, 1:-1] - p[:-2, 1:-1] - p[2:, 1:-1]
                              - p[1:-1, :-2] - p[1:-1, 2:])
            pAp = F.dot2d(p, Ap)
            alpha = rtr / pAp
            x[...] = x + alpha * p
            r[...] = r - alpha * Ap
            rtr_new = F.dot2d(r, r)
            beta[...] = rtr_new / rtr
            rtr[...] = rtr_new
            self.keep += [pAp, alpha, rtr_new]
        self.add_step(step)

        # start of a solve from a right-hand side that is already in `b` (uploaded with
        # cn_put / cn_put_local): x = 0, r = p = b, rtr = r.r
        def init():
            x[...] = 0.0
            r[...] = b
            p[...] = b
            beta[...] = 0.0
            t = F.dot2d(r, r)
            rtr[...] = t
            self.keep.append(t)
        self.init_blob = wire.dag_blob(_capture_step(init))


class Jacobi2D(Workload):
    name = "jacobi2d"
    metric = "jacobi2d_iterations_per_sec"

    @classmethod
    def describe(cls, nranks=1, scale=1.0):
        n = max(8, int(2048 * scale))
        shape = (n * nranks, n)
        return {"shape": shape, "points": shape[0] * n, "bytes_per_step": 16 * shape[0] * n,
                "description": (f"C1 Jacobi2D 5-point, {n}x{n} per GPU (global {shape[0]}x{n}), "
                                "residual sum((new-old)^2) every 10 iterations")}

    def __init__(self, interface, nranks=1, scale=1.0, res_every=10):
        super().__init__(interface, nranks, scale)
        self.res_every = res_every
        u = F.uniform(self.shape, seed=SEED + 1)
        u[0, :] = 1.0
        u[-1, :] = 0.0
        u[:, 0] = 0.0
        u[:, -1] = 0.0
        res = F.zeros((1,))
        F.execute(interface)
        self.u = u
        self.keep = [u, res]
        self.result = res

        def plain():
            u[1:-1, 1:-1] = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:])

        def with_residual():
            new = 0.25 * (u[:-2, 1:-1] + u[2:, 1:-1] + u[1:-1, :-2] + u[1:-1, 2:])
            d = new - u[1:-1, 1:-1]
            sq = d * d
            u[1:-1, 1:-1] = new
            s = F.sum_all(sq)
            del new, d, sq
            res[...] = s
            self.keep.append(s)
        self.add_step(plain)
        self.add_step(with_residual)

    def pick(self, i):
        return 1 if self.res_every and (i + 1) % self.res_every == 0 else 0


class Jacobi3D(Workload):
    name = "jacobi3d"
    metric = "jacobi3d_iterations_per_sec"

    @classmethod
    def describe(cls, nranks=1, scale=1.0):
        n = max(8, int(1024 * scale))
        shape = (n * nranks, n, n)
        return {"shape": shape, "points": shape[0] * n * n, "bytes_per_step": 16 * shape[0] * n * n,
                "description": (f"C5 Jacobi3D 7-point, {n}^3 per GPU (global {shape[0]}x{n}x{n}), "
                                "z-slab decomposition, residual every 10 iterations")}

    def __init__(self, interface, nranks=1, scale=1.0, res_every=10):
        super().__init__(interface, nranks, scale)
        self.res_every = res_every
        u = F.uniform(self.shape, seed=SEED + 5)
        u[0, :, :] = 1.0
        u[-1, :, :] = 0.0
        u[:, 0, :] = 0.0
        u[:, -1, :] = 0.0
        u[:, :, 0] = 0.0
        u[:, :, -1] = 0.0
        res = F.zeros((1,))
        F.execute(interface)
        self.u = u
        self.keep = [u, res]
        self.result = res
        c = 1.0 / 6.0

        def stencil():
            return c * (u[:-2, 1:-1, 1:-1] + u[2:, 1:-1, 1:-1] + u[1:-1, :-2, 1:-1]
                        + u[1:-1, 2:, 1:-1] + u[1:-1, 1:-1, :-2] + u[1:-1, 1:-1, 2:])

        def plain():
            u[1:-1, 1:-1, 1:-1] = stencil()

        def with_residual():
            new = stencil()
            d = new - u[1:-1, 1:-1, 1:-1]
            sq = d * d
            u[1:-1, 1:-1, 1:-1] = new
            s = F.sum_all(sq)
            del new, d, sq
            res[...] = s
            self.keep.append(s)
        self.add_step(plain)
        self.add_step(with_residual)

    def pick(self, i):
        return 1 if self.res_every and (i + 1) % self.res_every == 0 else 0


class Chain(Workload):
    name = "chain"
    metric = "fused_chain_repeats_per_sec"
    unit = "repeats/s"
    scaling = "strong"

    @classmethod
    def describe(cls, nranks=1, scale=1.0):
        n = max(8, int((1 << 28) * scale))
        return {"shape": (n,), "points": n, "bytes_per_step": 16 * n,
                "description": (f"C2 fused chain + sum, two float64 vectors of length {n} in total, "
                                "one fused kernel and one scalar result per repeat")}

    def __init__(self, interface, nranks=1, scale=1.0):
        super().__init__(interface, nranks, scale)
        n = self.shape[0]
        a = F.uniform((n,), seed=SEED + 2, low=-1.0, high=1.0)
        b = F.uniform((n,), seed=SEED + 22, low=-1.0, high=1.0)
        F.execute(interface)
        self.a, self.b = a, b
        self.keep = [a, b]

        def step():
            s = F.sum_all(F.exp(-a * a) * b + F.sqrt(F.absolute(a)) - 0.5 * b * b
                          + a / (1 + F.absolute(b)))
            self.result = s
        self.add_step(step)


class Matvec(Workload):
    name = "matvec"
    metric = "matvec_power_steps_per_sec"
    unit = "steps/s"
    scaling = "strong"

    @classmethod
    def describe(cls, nranks=1, scale=1.0):
        n = max(8, int(65536 * scale))
        return {"shape": (n, n), "points": n * n, "bytes_per_step": 8 * n * n + 3 * 8 * n,
                "description": (f"C4 dense row-partitioned matvec, A {n}x{n} float64, power iteration "
                                "y = A x; x = y / sqrt(y.y)")}

    def __init__(self, interface, nranks=1, scale=1.0):
        super().__init__(interface, nranks, scale)
        n = self.shape[0]
        A = F.uniform((n, n), seed=SEED + 4, low=-1.0 / 256, high=1.0 / 256)
        x = F.uniform((n,), seed=SEED + 44, low=-1.0, high=1.0)
        F.execute(interface)
        self.A, self.x = A, x
        self.keep = [A, x]

        def step():
            y = A @ x
            s = y @ y
            x[...] = y / F.sqrt(s)
            self.result = s
            self.keep += [y]
        self.add_step(step)


WORKLOADS = {w.name: w for w in (CG, Jacobi2D, Jacobi3D, Chain, Matvec)}
