"""Shared helpers: run one frontend program on the GPU backend and on the CPU oracle."""
import numpy as np

import charmnumeric_b200 as cnp
from charmnumeric_b200 import frontend as F
from oracle.oracle import Oracle


def run_oracle(fn):
    """Run ``fn`` (which builds lazy arrays and returns a dict name -> Array) on the CPU
    oracle only.  Returns dict name -> ndarray."""
    cnp.reset_frontend_state()
    outs = fn()
    orc = Oracle()
    F.execute(None, mirror=orc)
    return {k: np.array(orc.get(v.name)).reshape(v.shape) for k, v in outs.items()}


def run_both(interface, fn):
    """Run ``fn`` through the C ABI on the GPU and through the oracle on the same DAG.
    Returns (gpu, cpu): two dicts name -> ndarray."""
    cnp.reset_frontend_state()
    outs = fn()
    orc = Oracle()
    F.execute(interface, mirror=orc)
    gpu = {k: interface.context.get(v.name).reshape(v.shape) for k, v in outs.items()}
    cpu = {k: np.array(orc.get(v.name)).reshape(v.shape) for k, v in outs.items()}
    # release what the program left behind so that tests do not accumulate device memory
    for v in outs.values():
        del v
    return gpu, cpu


def assert_bit_exact(gpu, cpu):
    for k in cpu:
        a, b = gpu[k], cpu[k]
        assert a.dtype == b.dtype, k
        assert a.shape == b.shape, k
        same = a.view(np.uint8).reshape(-1) == b.view(np.uint8).reshape(-1)
        if not same.all():
            bad = np.argwhere(a != b)
            raise AssertionError(f"{k}: {len(bad)} elements differ, first at {bad[:3].tolist()}: "
                                 f"gpu={a[tuple(bad[0])]!r} cpu={b[tuple(bad[0])]!r}")


def assert_rel(gpu, cpu, rtol):
    for k in cpu:
        a, b = np.asarray(gpu[k], np.float64), np.asarray(cpu[k], np.float64)
        denom = np.maximum(np.abs(b), np.finfo(np.float64).tiny)
        err = np.max(np.abs(a - b) / denom) if a.size else 0.0
        scale = np.max(np.abs(b)) if b.size else 1.0
        err_n = np.max(np.abs(a - b)) / (scale if scale > 0 else 1.0) if a.size else 0.0
        assert min(err, err_n) <= rtol, f"{k}: relative error {min(err, err_n):.3e} > {rtol:.1e}"


class DryRunOracle(Oracle):
    """Oracle that also pushes every fusible node through the backend's host-side compiler
    (lowering, CUDA code generation, NVRTC for sm_100a) -- no GPU needed."""

    def __init__(self):
        super().__init__()
        self.compiled = 0

    def run(self, nodes, deletes=()):
        for n in nodes:
            if n.fusible:
                cnp.group_compile_check(n)
                self.compiled += 1
        super().run(nodes, deletes)


class OracleInterface:
    """Stand-in for CharmNumericInterface on machines without a GPU: the frontend executes
    on the oracle only.  Lets the reference-style tests run unchanged on CPU."""

    context = None

    def __init__(self, dry_run=True):
        self.mirror = DryRunOracle() if dry_run else Oracle()

    def get(self, ndims, name, size, dtype=None):
        return np.array(self.mirror.get(name)).reshape(-1)

    def connect(self, *args, **kwargs):
        return self

    def close(self):
        pass
