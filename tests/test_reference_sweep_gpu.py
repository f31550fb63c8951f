"""Differential sweep against the reference's own CUDA backend (oracle/_ref, see oracle/build_ref.py): the op / dtype
combinations that the reference's GPU-marked tests exercise (tests/ut/test_elemwise.py:22-330, test_cmp.py:24-120,
test_select.py, test_cast.py:25-165, test_broadcast.py, test_reduce.py:22-107) are built once per backend and run on
the same seeded inputs.  Integer / compare / select / cast / logical results must be identical bit for bit; floating
results agree within 1e-5 (fp32) or 1e-3 (fp16, the reference's own tolerance).  Skipped when oracle/_ref is absent."""
import numpy as np
import pytest

from oracle import ref_backend
from tests.util import TOL_EXACT, assert_close

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(ref_backend.module() is None, reason="oracle/_ref/_dvm_py was not built")]

F16, BF16, F32, I32, BOOL = 1, 2, 3, 4, 0


def both(build, arrays, dtypes=None, ours="vector", theirs="vector"):
    from dvm_b200.tester import Tester
    dtypes = dtypes or [None] * len(arrays)
    outs = []
    for k in (Tester(ours), ref_backend.RefKernel(theirs)):
        vals = build(k, *[k.load(a, d) for a, d in zip(arrays, dtypes)])
        vals = vals if isinstance(vals, (tuple, list)) else (vals,)
        stores = [k.store(v) for v in vals]
        k.run()
        outs.append([np.asarray(k.output(s)) for s in stores])
    return outs


def tol_of(dt):
    return 1e-3 if dt == np.float16 else 1e-5


@pytest.mark.parametrize("dt", [np.float16, np.float32])
@pytest.mark.parametrize("op", ["sqrt", "abs", "log", "exp", "reciprocal"])
def test_unary(dt, op):
    a = np.random.default_rng(1).uniform(0.1, 4.0, (32, 1024)).astype(dt)
    dev, ref = both(lambda k, x: getattr(k, op)(x), [a])
    assert_close(dev[0], ref[0], tol_of(dt), op)


@pytest.mark.parametrize("op", ["round", "floor", "ceil", "trunc"])
def test_rounding_fp32_exact(op):
    a = np.random.default_rng(2).normal(0, 20, (7, 333)).astype(np.float32)
    a[0, :8] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 0.0, -0.0]
    dev, ref = both(lambda k, x: getattr(k, op)(x), [a])
    assert_close(dev[0], ref[0], TOL_EXACT, op)


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_isfinite_exact(dt):
    a = np.random.default_rng(3).normal(0, 1, (16, 64)).astype(dt)
    a[0, :4] = [np.inf, -np.inf, np.nan, 0.0]
    dev, ref = both(lambda k, x: k.isfinite(x), [a])
    assert_close(dev[0], ref[0], TOL_EXACT, "isfinite")


@pytest.mark.parametrize("dt", [np.float16, np.float32])
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "maximum", "minimum"])
def test_binary(dt, op):
    rng = np.random.default_rng(4)
    a = rng.normal(0, 1, (1312, 131)).astype(dt)
    b = rng.uniform(0.5, 2.0, (1312, 131)).astype(dt)
    dev, ref = both(lambda k, x, y: k.copy(getattr(k, op)(k.copy(x), k.copy(y))), [a, b])
    assert_close(dev[0], ref[0], TOL_EXACT if op in ("add", "sub", "mul", "maximum", "minimum") else tol_of(dt), op)


@pytest.mark.parametrize("dt", [np.bool_, np.float16, np.float32])
@pytest.mark.parametrize("shape", [(1312, 131), (16, 11), (128, 777)])
def test_logical(dt, shape):
    rng = np.random.default_rng(5)
    a = rng.choice([True, False], shape).astype(dt)
    b = rng.choice([True, False], shape).astype(dt)
    dev, ref = both(lambda k, x, y: (k.logical_or(x, y), k.logical_and(x, y), k.logical_not(x)), [a, b])
    for d, r in zip(dev, ref):
        assert_close(d, r, TOL_EXACT, "logical %s" % (dt,))


def test_logical_of_mixed_compares():
    rng = np.random.default_rng(6)
    shape = (128, 777)
    a, b = (rng.integers(-1024, 1024, shape).astype(np.int32) for _ in range(2))
    c, d = (rng.normal(0, 1, shape).astype(np.float32) for _ in range(2))
    dev, ref = both(lambda k, x0, x1, x2, x3: (k.logical_or(k.greater(x0, x1), k.less(x2, x3)),
                                               k.logical_and(k.greater(x0, x1), k.less(x2, x3))), [a, b, c, d])
    for dd, rr in zip(dev, ref):
        assert_close(dd, rr, TOL_EXACT, "logical of compares")


@pytest.mark.parametrize("dt", [np.float16, np.float32])
def test_scalar_forms(dt):
    a = np.random.default_rng(7).normal(0.05, 1, (32, 1024)).astype(dt)

    def build(k, x):
        return (k.add(x, 0.1), k.mul(x, 0.1), k.div(x, 0.1), k.maximum(x, 0.1), k.minimum(x, 0.1), k.div(0.1, x),
                k.sub(0.1, x), k.sub(x, 0.1))

    dev, ref = both(build, [a])
    for d, r in zip(dev, ref):
        assert_close(d, r, tol_of(dt), "scalar forms")


@pytest.mark.parametrize("dt", [np.float16, np.float32, np.int32])
def test_compares_with_special_values(dt):
    rng = np.random.default_rng(8)
    a = rng.integers(-3, 3, (64, 257)).astype(dt)
    b = rng.integers(-3, 3, (64, 257)).astype(dt)
    if dt != np.int32:
        a[0, :3] = [np.nan, np.inf, -0.0]
        b[0, :3] = [1.0, np.inf, 0.0]
    names = ["equal", "not_equal", "greater", "greater_equal", "less", "less_equal"]
    dev, ref = both(lambda k, x, y: tuple(getattr(k, n)(x, y) for n in names) + (k.greater(x, 1), k.less_equal(1, x)), [a, b])
    for d, r, n in zip(dev, ref, names + ["greater scalar", "scalar less_equal"]):
        assert_close(d, r, TOL_EXACT, "%s %s" % (n, dt))


@pytest.mark.parametrize("dt", [np.float16, np.float32, np.int32])
def test_select(dt):
    rng = np.random.default_rng(9)
    a, b = (rng.integers(-50, 50, (33, 129)).astype(dt) for _ in range(2))
    c = rng.choice([True, False], (33, 129))
    dev, ref = both(lambda k, x, y, m: (k.select(m, x, y), k.select(k.greater(x, y), x, y)), [a, b, c])
    for d, r in zip(dev, ref):
        assert_close(d, r, TOL_EXACT, "select %s" % (dt,))


@pytest.mark.parametrize("src,dst", [(np.float16, F32), (np.float32, F16), (np.float16, I32), (np.int32, F32), (np.int32, F16),
                                     (np.float32, I32), (np.float32, BOOL), (np.float16, BOOL), (np.int32, BOOL), (np.bool_, F32),
                                     (np.float32, BF16)])
def test_casts(src, dst):
    rng = np.random.default_rng(10)
    a = (rng.normal(0, 100, (1024, 32)) if src != np.bool_ else rng.choice([True, False], (1024, 32))).astype(src)
    if src in (np.float16, np.float32):
        a[0, :4] = [0.0, -0.0, 0.5, -0.5]
    ours, theirs = both(lambda k, x: k.copy(k.cast(k.copy(x), dst)), [a])
    if dst == BF16:
        theirs[0] = np.asarray(theirs[0]).view(np.uint16)
        ours[0] = np.asarray(ours[0]).view(np.uint16)
    assert_close(ours[0], theirs[0], TOL_EXACT, "cast %s -> %d" % (src, dst))


def test_bf16_arithmetic():
    rng = np.random.default_rng(11)
    a, b = (rng.normal(0, 1, (64, 300)).astype(np.float32) for _ in range(2))
    ours, theirs = both(lambda k, x, y: k.cast(k.add(k.mul(x, y), y), F32), [a, b], dtypes=[BF16, BF16])
    assert_close(ours[0], theirs[0], TOL_EXACT, "bf16 mul/add rounded per op")


@pytest.mark.parametrize("shapes", [((64, 300), (300,)), ((64, 300), (64, 1)), ((5, 1, 33), (1, 7, 33)), ((1,), (17, 129))])
def test_broadcasting_binary(shapes):
    rng = np.random.default_rng(12)
    a, b = (rng.normal(0, 1, s).astype(np.float32) for s in shapes)
    dev, ref = both(lambda k, x, y: (k.add(x, y), k.greater(x, y)), [a, b])
    assert_close(dev[0], ref[0], TOL_EXACT, "broadcast add")
    assert_close(dev[1], ref[1], TOL_EXACT, "broadcast compare")


@pytest.mark.parametrize("shape,dims,keep", [((64, 300), (1,), True), ((64, 300), (1,), False), ((40, 33), (0,), False),
                                            ((5, 7, 64), (1, 2), True), ((3, 4, 5, 6), (0, 2), True), ((1000,), (0,), False)])
def test_reduce_sum(shape, dims, keep):
    a = np.random.default_rng(13).normal(0, 1, shape).astype(np.float32)
    dev, ref = both(lambda k, x: k.sum(x, dims, keep), [a])
    assert_close(dev[0], ref[0], 1e-4, "sum %s over %s" % (shape, dims))


def test_integer_ops_and_pow():
    rng = np.random.default_rng(14)
    i, j = (rng.integers(-30000, 30000, (17, 129)).astype(np.int32) for _ in range(2))
    x = rng.uniform(0.5, 2.0, (17, 129)).astype(np.float32)
    dev, ref = both(lambda k, a, b, c: (k.add(k.mul(a, b), 7), k.maximum(a, b), k.abs(a), k.pow(c, 3), k.pow(c, c)), [i, j, x])
    for d, r, what, tol in zip(dev, ref, ["int mul add", "int max", "int abs", "x^3", "x^x"], [0, 0, 0, 1e-5, 1e-5]):
        assert_close(d, r, tol, what)
