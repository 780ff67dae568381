"""Backend-generic lazy-graph cases: the reference's own fixtures
(ug-core/src/common_tests.rs, ug-core/tests/lb_tests.rs), written once and run
on the CPU oracle device (CPU suite) and on the B200 device (GPU suite)."""
import numpy as np

from ug_b200 import DType
from ug_b200.lazy import LB, BinaryOp as B, CompilationCache, ReduceOp as R, Schedule, UnaryOp as U

F = np.float32


def add(dev):           # common_tests.rs:6-13
    lb = LB.cst(40., (5, 2), dev).binary(B.Add, LB.cst(2., (5, 2), dev))
    assert np.array_equal(lb.data_vec(), np.full(10, 42., F))


def mm(dev):            # common_tests.rs:15-22
    lb = LB.cst(1., (4, 2), dev).matmul(LB.cst(2., (2, 3), dev))
    assert np.array_equal(lb.data_vec(), np.full(12, 4., F))


def cat(dev):           # common_tests.rs:24-35, including the pinned non-outer-axis behaviour
    a = [LB.copy(np.array(v, F), (2, 2), dev) for v in ([1., 2., 3., 4.], [1.1, 2.1, 3.1, 4.1], [1.2, 2.2, 3.2, 4.2])]
    assert np.array_equal(LB.cat(a, 0).data_vec(), np.array([1.0, 2.0, 3.0, 4.0, 1.1, 2.1, 3.1, 4.1, 1.2, 2.2, 3.2, 4.2], F))
    # axis 1: every piece is written with a contiguous layout at an element offset, so this is not a
    # concatenation; the reference pins the first 8 values (the last 4 are uninitialised memory that
    # happens to read 0 on its CPU backend)
    got = LB.cat(a, 1).data_vec()
    assert np.array_equal(got[:8], np.array([1.0, 2.0, 1.1, 2.1, 1.2, 2.2, 3.2, 4.2], F))


def schedule_one_kernel(dev):   # lb_tests.rs:4-28: cst + cst is a single kernel item
    lb = LB.cst(40., (5, 2), dev).binary(B.Add, LB.cst(2., (5, 2), dev))
    s = Schedule.create_one(lb)
    assert s.items() == ["Kernel"]
    text = s.ssa_text(0)        # default Opts: two nested sequential loops, one store
    assert text.count(": range ") == 2 and text.count("store.f32") == 1 and "thread_idx" not in text


def lb_copy(dev):       # lb_tests.rs:72-105: a compiled schedule re-runs on mutated inputs
    lhs = LB.copy(np.arange(6, dtype=F), (2, 3), dev)
    lb = lhs.binary(B.Add, LB.cst(2., (2, 3), dev)).binary(B.Mul, LB.cst(0.5, (2, 3), dev))
    sched = Schedule.create_one(lb).compile()
    sched.run()
    assert np.array_equal(lb.data_vec(), np.array([1.0, 1.5, 2.0, 2.5, 3.0, 3.5], F))
    lhs.write(np.array([0., 0., -8., 3., 4., -2.], F))
    sched.run()
    assert np.array_equal(lb.data_vec(), np.array([1.0, 1.0, -3.0, 2.5, 3.0, 0.0], F))


def schedule_broadcast(dev):    # lb_tests.rs:107-117
    lb = LB.cst(40., (5, 2), dev).binary(B.Add, LB.cst(2., (), dev).broadcast((5, 2)))
    assert np.array_equal(lb.data_vec(), np.full(10, 42., F))


def lb_layout(dev):     # lb_tests.rs:156-174
    lb = LB.copy(np.arange(6, dtype=F), (2, 3), dev).transpose(0, 1)
    assert np.array_equal(lb.data_vec(), np.array([0., 3., 1., 4., 2., 5.], F))
    lb = lb.transpose(0, 1).merge_dims(0)
    assert lb.dims() == (6,)
    assert np.array_equal(lb.data_vec(), np.arange(6, dtype=F))


def lb_set(dev):        # lb_tests.rs:207-229
    dst = LB.copy(np.arange(6, dtype=F), (2, 3), dev)
    src = dst.binary(B.Mul, dst)
    assert np.array_equal(src.data_vec(), np.array([0., 1., 4., 9., 16., 25.], F))
    assert np.array_equal(dst.data_vec(), np.arange(6, dtype=F))
    dst = dst.set(src)
    assert np.array_equal(dst.data_vec(), np.array([0., 1., 4., 9., 16., 25.], F))
    dst = dst.set_l(LB.copy(np.array([3., 1., 2.], F), (3,), dev), (3,))
    assert np.array_equal(dst.data_vec(), np.array([3., 1., 2., 9., 16., 25.], F))


def custom_ops(dev, add_one, add_one_ip):
    """lb_tests.rs:119-154 (custom) and :176-205 (custom_ip runs again on every realize)."""
    buf = LB.copy(np.arange(6, dtype=F), (2, 3), dev)
    lb = LB.custom(add_one, [buf], (2, 3), DType.F32, dev).binary(B.Mul, LB.cst(2., (2, 3), dev))
    sched = Schedule.create_one(lb).compile()
    sched.run()
    assert np.array_equal(lb.data_vec(), np.array([2., 4., 6., 8., 10., 12.], F))
    buf.write(np.array([0., 0., -8., 3., 4., -2.], F))
    sched.run()
    assert np.array_equal(lb.data_vec(), np.array([2., 2., -14., 8., 10., -2.], F))
    lb = LB.copy(np.arange(6, dtype=F), (2, 3), dev)
    lb = lb.custom_ip(add_one_ip, []).custom_ip(add_one_ip, []).custom_ip(add_one_ip, [])
    assert np.array_equal(lb.data_vec(), np.array([3., 4., 5., 6., 7., 8.], F))
    lb.write(np.array([3., 0., -8., 6., 7., -2.], F))
    assert np.array_equal(lb.data_vec(), np.array([6., 3., -5., 9., 10., 1.], F))


def errors(dev):
    from ug_b200 import UgError
    import pytest
    a, b = LB.cst(1., (2, 3), dev), LB.cst(1., (3, 2), dev)
    with pytest.raises(UgError, match="shape mismatch"):
        a.binary(B.Add, b)
    with pytest.raises(UgError, match="dtype mismatch"):
        a.binary(B.Add, LB.cst(1, (2, 3), dev))
    with pytest.raises(UgError, match="shape mismatch in matmul"):
        a.matmul(a)
    with pytest.raises(UgError, match="cannot reshape"):
        a.reshape((7,))
    with pytest.raises(UgError, match="cannot broadcast"):
        a.broadcast((2, 4))
    with pytest.raises(UgError, match="cannot squeeze"):
        a.squeeze(0)
    with pytest.raises(UgError, match="dim out of range"):
        a.reduce(R.Sum, 2)
    with pytest.raises(UgError, match="cannot narrow"):
        a.narrow(1, 2, 2)
    with pytest.raises(UgError, match="unexpected target sizes"):
        a.split_dim(1, 2, 2)
    with pytest.raises(UgError, match="set_l out of bounds"):
        a.set_l(LB.cst(1., (4,), dev), (4,), offset=3)


def graph_softmax(dev, x):      # ug-llama/src/model.rs:94-101
    from ug_b200 import llama_graph as G
    return G.softmax(LB.copy(x, x.shape, dev)).data_vec().reshape(x.shape)


def graph_rms_silu(dev, x, w, g, eps=1e-5):   # rms_norm(x) * w * silu(gate): one fused kernel (model.rs:65-78,103-109)
    from ug_b200 import llama_graph as G
    xs, ws, gs = LB.copy(x, x.shape, dev), LB.copy(w, w.shape, dev), LB.copy(g, g.shape, dev)
    lb = G.rms_norm(xs, ws, eps).binary(B.Mul, G.silu(gs))
    s = Schedule.create_one(lb)
    return lb.data_vec().reshape(x.shape), s.items()


def layout_chain(dev, x):
    """split_dim / transpose / narrow / merge_dims / broadcast chain against numpy (bit-exact copies)."""
    b, t, hd = x.shape
    h = 4
    lb = LB.copy(x, x.shape, dev).split_dim(2, h, hd // h).transpose(2, 1)        # [b, h, t, d]
    got = lb.narrow(2, 1, t - 1).merge_dims(-2).data_vec()                          # [b, h, (t-1)*d]
    ref = x.reshape(b, t, h, hd // h).transpose(0, 2, 1, 3)[:, :, 1:].reshape(b, h, -1)
    assert np.array_equal(got.reshape(ref.shape), ref)
    rep = lb.split_dim(1, h, 1).broadcast((b, h, 3, t, hd // h)).merge_dims(1)      # repeat, model.rs:80-92
    ref = np.repeat(x.reshape(b, t, h, hd // h).transpose(0, 2, 1, 3), 3, axis=1)
    assert np.array_equal(rep.data_vec().reshape(ref.shape), ref)


def cache_hits(dev):    # cache.rs: a structurally equal kernel compiles once; another shape misses
    cache = CompilationCache()
    for n in (8, 8, 12):
        x = LB.copy(np.arange(n, dtype=F), (n,), dev)
        Schedule.create_one(x.binary(B.Mul, x).unary(U.Sqrt)).compile(cache).run()
    assert (cache.misses, cache.hits) == (2, 1)
