"""Shape handling on the device against the expectations of the reference's GPU-marked shape tests, with seeded random
data instead of constant fills: reshape inside a fused graph (tests/ut/test_reshape.py:22-275), dynamic shapes re-read
at every run (tests/ut/test_dynamic_shape.py:66-162), tiles that do not divide the shape (tests/ut/test_unalign.py) and
broadcast forms (tests/ut/test_broadcast.py).  Every case is checked against the NumPy formula of the reference test under
that test's tolerance, and, when the reference's own CUDA backend was built into oracle/_ref, against its output as well.
"""
import numpy as np
import pytest

from oracle import ref_backend
from tests.util import assert_close

pytestmark = pytest.mark.gpu

HAVE_REF = ref_backend.module() is not None


def run(build, arrays, ker="vector", ref_ker="vector"):
    """Evaluates build(k, *loads) on this library and, when built, on the reference backend; returns ([ours], [theirs])."""
    from dvm_b200.tester import Tester
    outs = []
    for k in [Tester(ker)] + ([ref_backend.RefKernel(ref_ker)] if HAVE_REF else []):
        vals = build(k, *[k.load(a) for a in arrays])
        vals = vals if isinstance(vals, (tuple, list)) else (vals,)
        stores = [k.store(v) for v in vals]
        k.run()
        outs.append([np.asarray(k.output(s)) for s in stores])
    return outs[0], (outs[1] if HAVE_REF else None)


def check(ours, theirs, want, tol, what, ref_tol=None):
    for i, w in enumerate(want):
        assert_close(ours[i], w, tol, what + " against NumPy")
        if theirs is not None:
            assert_close(ours[i], theirs[i], tol if ref_tol is None else ref_tol, what + " against the reference backend")


@pytest.mark.parametrize("reduce_dims", [(2,), (1,)])
def test_broadcast_reshape_reduce(reduce_dims):
    # test_reshape.py:22-41
    b = np.random.default_rng(1).normal(0, 1, (10, 3, 1)).astype(np.float32)
    ours, theirs = run(lambda k, y: k.sum(k.reshape(k.broadcast(y, [10, 3, 4]), [1, 10, 12]), list(reduce_dims), True), [b])
    want = np.sum(np.broadcast_to(b, (10, 3, 4)).reshape(1, 10, 12), reduce_dims, keepdims=True)
    check(ours, theirs, [want], 1e-4, "broadcast -> reshape -> sum")


def test_unary_reshape_unary_and_cast():
    # test_reshape.py:44-71
    x = np.random.default_rng(2).uniform(1, 100, (16, 16)).astype(np.float32)
    ours, theirs = run(lambda k, a: (k.sqrt(k.reshape(k.sqrt(a), [32, 8])), k.cast(k.sqrt(k.reshape(k.sqrt(a), [32, 8])), 1)), [x])
    want = np.sqrt(np.sqrt(x)).reshape(32, 8)
    check(ours, theirs, [want, want.astype(np.float16)], 1e-5, "sqrt -> reshape -> sqrt", ref_tol=1e-5)


def test_select_with_reshaped_operand():
    # test_reshape.py:74-90
    rng = np.random.default_rng(3)
    a = rng.normal(0, 1, (9,)).astype(np.float32)
    b = rng.normal(0, 1, (3, 3)).astype(np.float32)
    c = rng.choice([True, False], (3, 3))
    ours, theirs = run(lambda k, m, y, z: k.select(m, k.reshape(y, [3, 3]), z), [c, a, b])
    check(ours, theirs, [np.where(c, a.reshape(3, 3), b)], 0, "select with a reshaped operand")


def test_broadcast_around_reshape():
    # test_reshape.py:93-126
    rng = np.random.default_rng(4)
    b = rng.normal(0, 1, (1, 8)).astype(np.float32)
    ours, theirs = run(lambda k, y: k.broadcast(k.reshape(k.broadcast(y, [10, 8]), [10, 1, 8]), [10, 4, 8]), [b])
    check(ours, theirs, [np.broadcast_to(np.broadcast_to(b, (10, 8)).reshape(10, 1, 8), (10, 4, 8))], 0, "broadcast-reshape-broadcast")
    b = rng.normal(0, 1, (10, 3, 4)).astype(np.float32)
    ours, theirs = run(lambda k, y: k.broadcast(k.reshape(y, [1, 10, 12]), [8, 10, 12]), [b])
    check(ours, theirs, [np.broadcast_to(b.reshape(1, 10, 12), (8, 10, 12))], 0, "reshape-broadcast")
    ours, theirs = run(lambda k: k.broadcast(k.reshape(k.full(0.3, [3, 10], 3), [3, 1, 10]), [3, 10, 10]), [])
    check(ours, theirs, [np.full((3, 10, 10), 0.3, np.float32)], 0, "full-reshape-broadcast")


def test_two_reshapes_of_one_input():
    # test_reshape.py:129-142
    a = np.random.default_rng(5).uniform(0.1, 1, (54, 89)).astype(np.float32)
    ours, theirs = run(lambda k, x: k.add(k.sqrt(k.reshape(x, [89, 54])), k.reshape(k.reciprocal(x), [89, 54])), [a])
    check(ours, theirs, [(np.sqrt(a) + np.reciprocal(a)).reshape(89, 54)], 1e-5, "two reshapes of one input")


def test_reshape_after_mixed_dtype_broadcast():
    # test_reshape.py:171-205
    rng = np.random.default_rng(6)
    a = rng.normal(0, 1, (1, 320)).astype(np.float16)
    b = np.asarray(rng.normal(0, 1, ()), dtype=np.float32)
    ours, theirs = run(lambda k, x1, x2: k.mul(k.reshape(k.cast(x1, 3), [320]), x2), [a, b])
    check(ours, theirs, [a.astype(np.float32).reshape(320) * b], 1e-5, "cast -> reshape -> mul by a 0-d tensor")
    for s1, s2, s3 in [((10, 20, 8), (20, 8), (200, 8)), ((10, 20, 8), (8,), (200, 8)), ((10, 20, 8), (8,), (10, 160))]:
        a = rng.normal(0, 1, s1).astype(np.float32)
        b = rng.normal(0, 1, s2).astype(np.float32)
        ours, theirs = run(lambda k, x1, x2: k.mul(k.reshape(k.add(x1, x2), list(s3)), 0.1), [a, b])
        check(ours, theirs, [(a + b).reshape(s3) * np.float32(0.1)], 1e-5, "add -> reshape %s -> mul" % (s3,))


def test_reduce_over_a_reshaped_leading_axis():
    # test_reshape.py:208-215
    a = np.random.default_rng(7).normal(-0.5, 0.5, (128, 1)).astype(np.float32)
    ours, theirs = run(lambda k, x: k.sum(k.reshape(x, [1, 128]), [1], True), [a])
    check(ours, theirs, [np.sum(a, (0,), keepdims=True).reshape(1, 1)], 1e-4, "reshape -> sum")


@pytest.mark.parametrize("s1,s2", [((2, 3, 64), (2, 6, 32)), ((1000, 4), (100, 40)), ((128,), (128, 1)), ((1000, 4), (20, 5, 40)),
                                   ((3, 1000, 4), (3, 20, 5, 40)), ((3, 20, 5, 4, 2), (3, 10, 40, 2)), ((3, 2, 10, 64), (6, 10, 16, 4)),
                                   ((3, 2, 1, 10), (6, 1, 10)), ((3, 2, 1, 1, 10), (6, 1, 10)), ((3, 2, 1, 10), (6, 1, 1, 10))])
def test_reshape_between_elementwise_ops(s1, s2):
    # test_reshape.py:218-275
    a = np.random.default_rng(8).normal(0, 1, s1).astype(np.float32)
    ours, theirs = run(lambda k, x: (k.add(k.reshape(k.mul(x, 0.6), list(s2)), 0.1), k.reshape(k.mul(x, 0.6), list(s2))), [a])
    y = (a * np.float32(0.6)).reshape(s2)
    check(ours, theirs, [y + np.float32(0.1), y], 1e-5, "mul -> reshape %s -> add" % (s2,))


@pytest.mark.parametrize("sa,sb,sc,dims", [((10, 64), (10, 1), (2, 5, 64), (1,)), ((10, 64), (10, 1), (10, 4, 16), (2,)),
                                           ((10, 4, 64), (10, 4, 1), (10, 32, 8), (0,)), ((2, 10, 64), (64,), (20, 64), (1,)),
                                           ((10, 4, 64), (10, 4, 1), (10, 32, 8), (1,))])
def test_add_reshape_reduce(sa, sb, sc, dims):
    # test_reshape.py:278-298
    rng = np.random.default_rng(9)
    a = rng.normal(0, 0.3, sa).astype(np.float32)
    b = rng.normal(0, 0.2, sb).astype(np.float32)
    ours, theirs = run(lambda k, x1, x2: k.sum(k.reshape(k.add(x1, x2), list(sc)), list(dims), True), [a, b])
    check(ours, theirs, [np.sum((a + b).reshape(sc), axis=dims, keepdims=True)], 1e-4, "add -> reshape -> sum %s" % (dims,))


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_row_broadcast_over_odd_width(dt):
    # test_unalign.py:22-33 and :65-75
    rng = np.random.default_rng(10)
    a = rng.normal(0, 1, (16, 1)).astype(dt)
    b = rng.normal(0, 1, (16, 41)).astype(dt)
    ours, theirs = run(lambda k, x, y: k.add(x, y), [a, b])
    check(ours, theirs, [a + b], 0, "[16,1] + [16,41] %s" % (dt,))
    c = rng.normal(0, 1, (4080,)).astype(np.float32)
    ours, theirs = run(lambda k, x: k.add(x, 0.3), [c])
    check(ours, theirs, [c + np.float32(0.3)], 0, "[4080] + scalar")


# ---- dynamic shapes: one compiled graph, shapes and axis lists re-read at every run --------------------------------------

def test_dynamic_reshape_and_implicit_broadcast():
    # test_dynamic_shape.py:22-63
    from dvm_b200.tester import Tester
    rng = np.random.default_rng(11)
    t = Tester("vector:dyn")
    x, y = t.load([-1], "float32"), t.load([-1], "float32")
    ref = t.int_array()
    out = t.store(t.add(t.reshape(x, ref), y))
    for xs, rs, ys in [((10,), (2, 5), (2, 5)), ((20, 40), (800, 1), (800, 16)), ((2, 40), (1, 80, 1), (10, 80, 32))]:
        xd, yd = rng.normal(0, 1, xs).astype(np.float32), rng.normal(0, 1, ys).astype(np.float32)
        t.input(x, xd)
        t.input(y, yd)
        ref.update(list(rs))
        t.run()
        assert_close(t.output(out), xd.reshape(rs) + yd, 0, "dynamic reshape %s" % (rs,))
    t = Tester("vector:dyn")
    x, y = t.load([-1], "float32"), t.load([-1], "float32")
    out = t.store(t.mul(t.add(x, 0.15), y))
    for xs, ys in [((1000,), (1000,)), ((500, 1), (500, 1024)), ((500, 1), (1, 1024)), ((4, 1, 12, 1), (4, 32, 12, 64))]:
        xd, yd = rng.normal(0, 1, xs).astype(np.float32), rng.normal(0, 1, ys).astype(np.float32)
        t.input(x, xd)
        t.input(y, yd)
        t.run()
        assert_close(t.output(out), (xd + np.float32(0.15)) * yd, 0, "dynamic broadcast %s x %s" % (xs, ys))


def test_dynamic_reduce_axes():
    # test_dynamic_shape.py:66-95
    from dvm_b200.tester import Tester
    rng = np.random.default_rng(12)
    t = Tester("vector:dyn")
    x = t.load([-1], "float32")
    dims = t.int_array()
    out = t.store(t.sum(x, dims, True))
    for xs, ds in [((10, 64), (1,)), ((12, 128), (0, 1)), ((3, 12, 20, 100), (1, 3))]:
        d = rng.normal(0, 1, xs).astype(np.float32)
        t.input(x, d)
        dims.update(list(ds))
        t.run()
        assert_close(t.output(out), np.sum(d, ds, keepdims=True), 1e-4, "dynamic sum over %s" % (ds,))
    t = Tester("vector:dyn")
    x = t.load([-1, 2, 4, 3000], "float32")
    out = t.store(t.sum(x, [0, 2], True))
    d = rng.normal(0, 1, (2, 2, 4, 3000)).astype(np.float32)
    for _ in range(3):
        t.input(x, d)
        t.run()
        assert_close(t.output(out), np.sum(d, (0, 2), keepdims=True), 1e-4, "sum over (0, 2) of [-1,2,4,3000]")


def test_dynamic_cast_chain_reduce_and_broadcast():
    # test_dynamic_shape.py:98-131
    from dvm_b200.tester import Tester
    rng = np.random.default_rng(13)
    t = Tester("vector:dyn")
    a = t.load([3, 1280, -1, -1], "float32")
    out = t.store(t.sum(t.cast(t.add(t.cast(a, "float16"), 0.1), "float32"), [0, 2, 3], True))
    for shape in [(3, 1280, 38, 36), (3, 1280, 44, 22)]:
        ax = rng.normal(0, 0.1, shape).astype(np.float32)
        t.input(a, ax)
        t.run()
        want = np.sum((ax.astype(np.float16) + np.float16(0.1)).astype(np.float32), (0, 2, 3), keepdims=True)
        assert_close(t.output(out), want, 1e-4, "cast chain -> sum %s" % (shape,))
    t = Tester("vector:dyn")
    x = t.load([-1], "float32")
    shape = t.int_array()
    out = t.store(t.mul(t.broadcast(x, shape), t.full(0.2, shape, "float32")))
    for xs, bs in [((1,), (10, 100)), ((1, 4, 1), (8, 4, 40))]:
        xd = rng.normal(0, 1, xs).astype(np.float32)
        t.input(x, xd)
        shape.update(list(bs))
        t.run()
        assert_close(t.output(out), np.broadcast_to(xd, bs) * np.float32(0.2), 0, "dynamic broadcast to %s" % (bs,))


def test_dynamic_three_outputs_with_row_sums():
    # test_dynamic_shape.py:134-162 (fp16 add -> fp32 -> square -> sum over the last axis, T = 2685..2687); rows cut to 300
    from dvm_b200.tester import Tester
    rng = np.random.default_rng(14)
    t = Tester("vector:dyn")
    p0, p1 = t.load([-1], "float16"), t.load([-1], "float16")
    y0 = t.add(p0, p1)
    out0 = t.store(y0)
    y1 = t.cast(y0, "float32")
    out1 = t.store(y1)
    out2 = t.store(t.sum(t.mul(y1, y1), [2], True))
    for rows in (2685, 300, 301):
        xd = rng.normal(0, 1, (1, rows, 4096)).astype(np.float16)
        yd = rng.normal(0, 1, (1, rows, 4096)).astype(np.float16)
        t.input(p0, xd)
        t.input(p1, yd)
        t.run()
        s = xd + yd
        assert_close(t.output(out0), s, 0, "fp16 sum")
        assert_close(t.output(out1), s.astype(np.float32), 0, "fp16 -> fp32")
        assert_close(t.output(out2), np.sum(s.astype(np.float32) ** 2, 2, keepdims=True), 1e-4, "row sums of squares")
