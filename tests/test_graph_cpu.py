"""Host-side logic of the lazy graph that needs no device: the execution order of Tensor::resolve
(tensor.rs:696-740) on a graph built from device-less leaves."""
import ctypes as C

import pytest


def _leaf(lib, capi, shape, dt=None):
    t = capi.describe(capi.F32 if dt is None else dt, shape, 0x1000)    # never dereferenced: the graph is not resolved
    h = C.c_void_p()
    assert lib.rcu_lazy_wrap(None, C.byref(t), C.byref(h)) == capi.OK
    return h


def _order(lib, capi, root):
    n = C.c_uint32()
    ids = (C.c_uint64 * 64)()
    assert lib.rcu_lazy_execution_order(root, ids, 64, C.byref(n)) == capi.OK
    return [ids[i] for i in range(n.value)]


def test_execution_order_visits_leaves_first():
    """out = (a + b) * c with a, b, c leaves, then out2 = relu(out) + d.

    The reference visits a node's sources leaves first and the sources that have sources of their own after
    them (`partition(|s| s.op().srcs().is_empty())` puts the leaves in the first list), each group in the order
    the op lists them; a node follows all of its sources."""
    from ratchet_b200 import capi
    lib = capi.lib()
    a, b, c, d = (_leaf(lib, capi, (4, 8)) for _ in range(4))
    s, m, r, o = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    assert lib.rcu_lazy_binary(0, a, b, C.byref(s)) == capi.OK          # s = a + b
    assert lib.rcu_lazy_binary(2, s, c, C.byref(m)) == capi.OK          # m = s * c      (sources: s has deps, c is a leaf)
    assert lib.rcu_lazy_unary(8, m, C.byref(r)) == capi.OK              # r = relu(m)
    assert lib.rcu_lazy_binary(0, r, d, C.byref(o)) == capi.OK          # o = r + d      (sources: r has deps, d is a leaf)
    ident = {name: lib.rcu_lazy_id(h) for name, h in dict(a=a, b=b, c=c, d=d, s=s, m=m, r=r, o=o).items()}
    got = _order(lib, capi, o)
    name_of = {v: k for k, v in ident.items()}
    # o: leaf d first, then r; r -> m; m: leaf c first, then s; s: a, b
    assert [name_of[i] for i in got] == ["d", "c", "a", "b", "s", "m", "r", "o"]
    # a shared source appears once, where it is first needed
    t = C.c_void_p()
    assert lib.rcu_lazy_binary(2, s, s, C.byref(t)) == capi.OK
    assert [name_of.get(i, "t") for i in _order(lib, capi, t)] == ["a", "b", "s", "t"]
    # a graph without a device can be inspected but not resolved
    assert lib.rcu_lazy_resolve(o) == capi.ERR_INVALID_ARG
    for h in (t, o, r, m, s, a, b, c, d):
        lib.rcu_lazy_release(h)


def test_builders_validate_without_a_device():
    from ratchet_b200 import capi
    lib = capi.lib()
    a = _leaf(lib, capi, (4, 8))
    b = _leaf(lib, capi, (3, 8))
    out = C.c_void_p()
    assert lib.rcu_lazy_binary(0, a, b, C.byref(out)) == capi.ERR_INVALID_ARG      # BroadcastingFailed (tensor.rs:258-261)
    h = _leaf(lib, capi, (4, 8), capi.F16)
    assert lib.rcu_lazy_binary(0, a, h, C.byref(out)) == capi.ERR_INVALID_ARG      # dtype mismatch
    for t in (a, b, h):
        lib.rcu_lazy_release(t)
