"""GPU tests of the slab-wise and executor-level entry points: cn_put_local, cn_get_root and
cn_execute_node, each through the C ABI, against NumPy / the oracle."""
import numpy as np
import pytest

from charmnumeric_b200 import wire
from oracle.oracle import Oracle

pytestmark = pytest.mark.gpu


def test_put_local_get_root_roundtrip(interface):
    ctx = interface.context
    rng = np.random.default_rng(7)
    host = rng.uniform(-1.0, 1.0, (37, 19))
    ctx.put_local(7001, host.shape, host)         # one rank: the slab is the whole array
    back = ctx.get_root(7001, root=0)
    assert back.tobytes() == host.tobytes()
    (b, e), slab = ctx.get_local(7001)
    assert (b, e) == (0, 37) and slab.tobytes() == host.tobytes()
    out = np.empty_like(host)
    assert ctx.get_local_into(7001, out) == (0, 37)
    assert out.tobytes() == host.tobytes()
    ctx.delete_array(7001)


def test_put_local_rejects_short_buffer(interface):
    from charmnumeric_b200._lib import CnError
    ctx = interface.context
    with pytest.raises(CnError) as err:
        ctx.put_local(7002, (8, 8), np.zeros((4, 8)))
    assert err.value.status == 1


def test_execute_node_runs_one_group_and_one_reduction(interface):
    ctx = interface.context
    rng = np.random.default_rng(8)
    a = rng.uniform(-1.0, 1.0, (33, 21))
    b = rng.uniform(-1.0, 1.0, (33, 21))
    ctx.put(7010, a)
    ctx.put(7011, b)
    la, lb = wire.leaf(7010, a.shape), wire.leaf(7011, b.shape)
    group = wire.Node(0, [
        wire.Ast(7012, wire.OP_MUL, is_temp=True, shape=a.shape, operands=[(la, None), (lb, None)]),
        wire.Ast(7013, wire.OP_ADD, shape=a.shape, operands=[(wire.Ref(7012), None), (la, None)]),
    ], fusible=True)
    dot = wire.Node(1, [wire.Ast(7014, wire.OP_REDUCE, shape=(1,), operands=[(la, None), (lb, None)])],
                    fusible=False)
    ctx.execute_node(group)
    ctx.execute_node(dot)
    orc = Oracle()
    orc.put(7010, a)
    orc.put(7011, b)
    orc.run([group, dot])
    assert ctx.get(7013).tobytes() == np.array(orc.get(7013)).tobytes()
    got, want = float(ctx.get(7014)[0]), float(orc.get(7014)[0])
    assert abs(got - want) <= 1e-10 * abs(want)
    for name in (7010, 7011, 7013, 7014):
        ctx.delete_array(name)


def test_execute_node_rejects_garbage(interface):
    from charmnumeric_b200._lib import CnError
    with pytest.raises(CnError):
        interface.context._check(interface.context._lib.cn_execute_node(interface.context._h, b"\x01\x02\x03", 3))
