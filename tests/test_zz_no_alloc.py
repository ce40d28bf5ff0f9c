"""GPU test of cn_dot_noalloc, the dot product for callers that cannot allocate device
memory (its scratch is a fixed array inside the library instead of an allocated buffer).

The test hands the entry point raw device pointers (torch owns the memory here, as such a
caller's own arena would), calls it twice in a row -- the second call finds the scratch as
the first one left it -- and compares each result with the CPU oracle's dot product of the
same host arrays and, as a second check, with what the regular path (a REDUCE node through
cn_receive_dag, read back with cn_get) gives for the same data, both within the tolerance the
reduction tests use.  A first call with n = 0 plays the warm-up a caller makes while memory
is still available (it loads the library's device image and resolves the scratch address).  Collected last on purpose (file name), so a failure
here cannot hide the result of any other test; it needs nothing from the tests before it.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
RTOL = 1e-10


def _regular_dot(ctx, name_a, name_b, name_out, a, b):
    from charmnumeric_b200 import wire
    ctx.put(name_a, a)
    ctx.put(name_b, b)
    node = wire.Node(0, [wire.Ast(name_out, wire.OP_REDUCE, shape=(1,), operands=[
        (wire.leaf(name_a, a.shape), None), (wire.leaf(name_b, b.shape), None)])], fusible=False)
    ctx.run([node])
    return float(ctx.get(name_out)[0])


@pytest.mark.parametrize("n", [1, 8191, 8192, 100003, 3_000_001])
def test_dot_noalloc_matches_regular_dot_twice(n):
    import torch
    from charmnumeric_b200 import Context, _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    from oracle import oracle as O
    ctx = Context(device=0)
    try:
        warm = torch.full((1,), float("nan"), dtype=torch.float64, device="cuda")
        assert lib.cn_dot_noalloc(C.c_void_p(warm.data_ptr()), C.c_void_p(warm.data_ptr()), 0,
                                  C.c_void_p(warm.data_ptr()), None) == 0
        torch.cuda.synchronize()
        assert float(warm.cpu()[0]) == 0.0
        for call in range(2):
            rng = np.random.default_rng(100 + call)
            a = rng.uniform(-1.0, 1.0, n)
            b = rng.uniform(-1.0, 1.0, n)
            want = float(O.dot(a, b))
            regular = _regular_dot(ctx, 9100, 9101, 9102, a, b)
            ta = torch.from_numpy(a).cuda()
            tb = torch.from_numpy(b).cuda()
            out = torch.full((1,), float("nan"), dtype=torch.float64, device="cuda")
            torch.cuda.synchronize()
            status = lib.cn_dot_noalloc(C.c_void_p(ta.data_ptr()), C.c_void_p(tb.data_ptr()), n,
                                        C.c_void_p(out.data_ptr()), None)
            assert status == 0
            torch.cuda.synchronize()
            got = float(out.cpu()[0])
            assert abs(got - want) <= RTOL * max(abs(want), 1e-300) + 1e-300, (n, call, got, want)
            assert abs(got - regular) <= RTOL * max(abs(want), 1e-300) + 1e-300, (n, call, got, regular)
    finally:
        ctx.close()


def test_dot_noalloc_rejects_oversize_and_bad_arguments():
    import torch
    from charmnumeric_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    x = torch.zeros(8, dtype=torch.float64, device="cuda")
    p = C.c_void_p(x.data_ptr())
    limit = 268435456
    assert lib.cn_dot_noalloc(p, p, limit + 1, p, None) == 13   # CN_STATUS_LIMIT, nothing launched
    assert lib.cn_dot_noalloc(None, p, 8, p, None) == 1
    assert lib.cn_dot_noalloc(p, p, -1, p, None) == 1
    torch.cuda.synchronize()
