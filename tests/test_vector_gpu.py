"""Device parity of the vector interpreter against the NumPy oracle (through the C ABI)."""
import numpy as np
import pytest

from dvm_b200 import workloads as W
from tests.util import BF16, TOL_EXACT, TOL_FP32, TOL_HALF, TOL_REDUCE, assert_close, run_both

pytestmark = pytest.mark.gpu

SHAPES = [(1,), (7,), (17, 129), (1312, 131), (2048,), (3, 5, 64), (257, 1024)]


@pytest.mark.parametrize("shape", SHAPES)
def test_fused_elementwise_shapes(shape):
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, shape).astype(np.float32)
    y = rng.uniform(-1, 1, shape).astype(np.float32)
    dev, ref, _ = run_both(W.fused_elementwise, [x, y])
    assert_close(dev[0], ref[0], TOL_FP32, "exp(x)*y+0.5 %s" % (shape,))


def test_config1_slice_bitwise_ops():
    # add/mul/sub are IEEE-exact on both sides; a division that feeds a compare stays IEEE-exact too, one that only
    # feeds arithmetic and stores may use the 2-ulp fast form
    rng = np.random.default_rng(1)
    x = rng.uniform(-1, 1, (300, 1000)).astype(np.float32)
    y = rng.uniform(0.5, 2, (300, 1000)).astype(np.float32)
    dev, ref, _ = run_both(lambda k, a, b: k.add(k.sub(k.mul(a, b), a), b), [x, y])
    assert_close(dev[0], ref[0], TOL_EXACT, "exact fp32 chain")
    dev, ref, t = run_both(lambda k, a, b: (k.div(a, b), k.greater(k.div(a, b), 0.25)), [x, y])
    assert "DivFast" in t.das() and "Div.fp32" in t.das()
    assert_close(dev[0], ref[0], TOL_FP32, "fast division")
    assert_close(dev[1], ref[1], TOL_EXACT, "compare of an exact division")


@pytest.mark.parametrize("dt", [np.float16, "bf16", np.float32])
def test_unary_chain(dt):
    rng = np.random.default_rng(2)
    x = rng.uniform(0.1, 4, (513, 77)).astype(np.float32)
    if dt == "bf16":
        xs, dts = x, [2]
    else:
        xs, dts = x.astype(dt), [None]
    dev, ref, _ = run_both(lambda k, a: k.abs(k.log(k.sqrt(k.exp(a)))), [xs], dtypes=dts)
    assert_close(dev[0], ref[0], TOL_FP32 if dt == np.float32 else TOL_HALF, "unary chain")


@pytest.mark.parametrize("op", ["round", "floor", "ceil", "trunc"])
def test_rounding_ops_exact(op):
    rng = np.random.default_rng(3)
    x = (rng.uniform(-8, 8, (1000,)) * 2).round() / 4
    x = x.astype(np.float32)
    dev, ref, _ = run_both(lambda k, a: getattr(k, op)(a), [x])
    assert_close(dev[0], ref[0], TOL_EXACT, op)


def test_broadcast_row_and_column():
    rng = np.random.default_rng(4)
    a = rng.normal(size=(64, 1)).astype(np.float32)
    b = rng.normal(size=(1, 200)).astype(np.float32)
    c = rng.normal(size=(64, 200)).astype(np.float32)
    dev, ref, _ = run_both(lambda k, x, y, z: k.add(k.mul(x, y), z), [a, b, c])
    assert_close(dev[0], ref[0], TOL_EXACT, "row/col broadcast")


def test_compare_select_cast_bit_exact():
    rng = np.random.default_rng(5)
    a = rng.normal(size=(333, 65)).astype(np.float32)
    b = rng.normal(size=(333, 65)).astype(np.float32)
    a[::7] = np.nan
    b[::11] = np.inf

    def build(k, x, y):
        m = k.greater(x, y)
        s = k.select(m, x, y)
        i = k.cast(k.mul(s, 100.0), 4)      # -> int32 (truncation)
        f16 = k.cast(x, 1)
        return m, s, k.cast(k.minimum(k.maximum(x, -1e4), 1e4), 4), f16, k.less_equal(f16, 0.25)

    dev, ref, _ = run_both(build, [np.nan_to_num(a, nan=0.5), b.clip(-10, 10)])
    for d, r, name in zip(dev, ref, ["mask", "select", "int", "f16", "cmp f16"]):
        assert_close(d, r, TOL_EXACT, name)


def test_compare_with_nan_inputs():
    a = np.array([np.nan, 1.0, -0.0, np.inf, 2.0, np.nan], np.float32)
    b = np.array([1.0, np.nan, 0.0, np.inf, 1.0, np.nan], np.float32)

    def build(k, x, y):
        return (k.equal(x, y), k.not_equal(x, y), k.greater(x, y), k.less_equal(x, y),
                k.maximum(x, y), k.minimum(x, y), k.isfinite(x))

    dev, ref, _ = run_both(build, [a, b])
    for d, r in zip(dev, ref):
        assert_close(d, r, TOL_EXACT, "nan compare")


def test_int32_ops_wrap():
    rng = np.random.default_rng(6)
    a = rng.integers(-2**31, 2**31 - 1, (4099,), dtype=np.int64).astype(np.int32)
    b = rng.integers(-2**31, 2**31 - 1, (4099,), dtype=np.int64).astype(np.int32)

    def build(k, x, y):
        return k.add(x, y), k.sub(x, y), k.mul(x, 3), k.maximum(x, y), k.abs(x), k.less(x, y), k.equal(x, 7)

    dev, ref, _ = run_both(build, [a, b])
    for d, r in zip(dev, ref):
        assert_close(d, r, TOL_EXACT, "int32")


def test_logical_ops_on_bool():
    rng = np.random.default_rng(7)
    a = rng.integers(0, 2, (1000,)).astype(np.bool_)
    b = rng.integers(0, 2, (1000,)).astype(np.bool_)
    dev, ref, _ = run_both(lambda k, x, y: (k.logical_and(x, y), k.logical_or(x, y), k.logical_not(x)), [a, b])
    for d, r, want in zip(dev, ref, [a & b, a | b, ~a]):
        assert_close(d, r, TOL_EXACT, "logical")
        assert_close(d, want, TOL_EXACT, "logical vs numpy")


@pytest.mark.parametrize("rows,cols", [(1, 4096), (7, 4096), (128, 4096), (33, 100), (5, 8), (16, 2048), (3, 5000)])
def test_rmsnorm_swiglu(rows, cols):
    rng = np.random.default_rng(3)
    h, r, g, u = (rng.normal(size=(rows, cols)).astype(np.float32) for _ in range(4))
    w = rng.normal(1, 0.02, size=(cols,)).astype(np.float32)
    dev, ref, _ = run_both(lambda k, *t: W.rmsnorm_swiglu(k, *t, cols), [h, r, w, g, u], ker_type="vector:spec,dyn",
                           dtypes=[2] * 5)
    assert_close(dev[0], ref[0], TOL_HALF, "rmsnorm")
    assert_close(dev[1], ref[1], TOL_HALF, "swiglu")


@pytest.mark.parametrize("shape", [(4, 8, 6, 6), (16, 32, 14, 14), (8, 3, 5, 7), (32, 8, 56, 56), (42, 5, 56, 56), (70, 3, 56, 56)])
def test_batchnorm(shape):
    rng = np.random.default_rng(2)
    n, c, hh, ww = shape
    x = rng.normal(size=shape).astype(np.float16)
    gamma = rng.normal(1, 0.1, size=(1, c, 1, 1)).astype(np.float32)
    beta = rng.normal(0, 0.1, size=(1, c, 1, 1)).astype(np.float32)
    dev, ref, _ = run_both(lambda k, a, g, b: W.batchnorm_train(k, a, g, b, n * hh * ww), [x, gamma, beta])
    assert_close(dev[0], ref[0], TOL_HALF, "bn y")
    assert_close(dev[1], ref[1], TOL_REDUCE, "bn mean")
    assert_close(dev[2], ref[2], TOL_REDUCE, "bn var")
    # against the plain NumPy formula as well
    xf = x.astype(np.float32)
    assert_close(dev[1].reshape(-1), xf.mean(axis=(0, 2, 3)), 1e-3, "mean vs numpy")
    assert_close(dev[2].reshape(-1), xf.var(axis=(0, 2, 3)), 1e-3, "var vs numpy")


@pytest.mark.parametrize("shape,dims,keep", [((64, 300), (1,), True), ((64, 300), (1,), False), ((5, 7, 64), (1, 2), True),
                                            ((1000,), (0,), False), ((3, 4, 5, 6), (0, 2), True), ((40, 33), (0,), False)])
def test_reduce_sum_patterns(shape, dims, keep):
    rng = np.random.default_rng(8)
    x = rng.normal(size=shape).astype(np.float32)
    dev, ref, _ = run_both(lambda k, a: k.sum(a, dims, keep), [x])
    assert_close(dev[0], ref[0], 1e-4, "sum %s over %s" % (shape, dims))


def test_softmax_max_and_sum():
    rng = np.random.default_rng(9)
    x = rng.normal(size=(77, 515)).astype(np.float32)

    def build(k, a):
        m = k.max(a, (1,), True)
        e = k.exp(k.sub(a, m))
        return k.div(e, k.sum(e, (1,), True))

    dev, ref, _ = run_both(build, [x])
    assert_close(dev[0], ref[0], 1e-4, "softmax")


def test_zero_size_shape_launches_nothing():
    from dvm_b200.tester import Tester
    t = Tester("vector")
    a = t.load(np.zeros((0, 16), np.float32))
    s = t.store(t.add(a, 1.0))
    t.run()
    assert t.output(s).shape == (0, 16)


def test_scalar_ref_and_relaunch():
    from dvm_b200.tester import Tester
    t = Tester("vector:dyn")
    x = np.arange(1000, dtype=np.float32)
    a = t.load(x)
    sc = t.scalar()
    s = t.store(t.mul(a, sc))
    for v in (2.0, -0.5):
        t.input(sc, v)
        t.run()
        assert_close(t.output(s), x * np.float32(v), TOL_EXACT, "scalar ref")


@pytest.mark.parametrize("mask", [1, 0])
@pytest.mark.parametrize("shape", [(1024, 32), (127,), (100, 100), (23, 23), (5231,)])
def test_element_any(mask, shape):
    # Kernel::ElemAny (include/dvm.h:496; tests/ut/test_element_any.py): 1 when any element differs from 0
    from dvm_b200.tester import Tester
    a = np.full(shape, mask, np.float32)
    t = Tester("vector")
    b = t.store(t.element_any(t.load(a)))
    t.run()
    assert t.output(b).shape == (1,) and t.output(b)[0] == mask
    a = np.zeros(shape, np.float16)
    a.reshape(-1)[a.size // 3] = -0.5 if mask else 0.0
    t = Tester("vector")
    b = t.store(t.element_any(t.abs(t.load(a))))
    t.run()
    assert t.output(b)[0] == mask
