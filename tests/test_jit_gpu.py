"""The ``@kernel`` decorator on the device, through the reference's import name (``import dvm``): the call contract of
python/dvm/jit.py as its examples use it (examples/01_add.py:19-37 with broadcasting inputs on a second call,
examples/02_batchnorm.py:25-60 with several results, a static-shape kernel, scalar arguments)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_bare_decorator_is_a_dynamic_split_kernel():
    import dvm

    @dvm.kernel
    def my_add(k, x, y):
        return k.store(k.add(k.load(x, dvm.float32), k.load(y, dvm.float32)))

    x = np.full([32, 32], 0.1, np.float32)
    y = np.full([32, 32], 0.3, np.float32)
    np.testing.assert_allclose(my_add(x, y), x + y, rtol=1e-6)
    x = np.full([32, 1], 0.2, np.float32)
    y = np.random.default_rng(0).standard_normal((32, 512)).astype(np.float32)
    np.testing.assert_allclose(my_add(x, y), x + y, rtol=1e-6)     # new shapes, broadcasting: planned again


def test_several_results_and_static_shapes():
    import dvm
    from dvm_b200 import workloads as W
    shape = (8, 16, 14, 14)

    @dvm.kernel("split", dynamic=False)
    def bn(k, x, g, b):
        xs = k.load(x, dvm.float16, shape)
        gs = k.load(g, dvm.float32, (1, 16, 1, 1))
        bs = k.load(b, dvm.float32, (1, 16, 1, 1))
        return [k.store(v) for v in W.batchnorm_train(k, xs, gs, bs, 8 * 14 * 14)]

    rng = np.random.default_rng(2)
    x = rng.standard_normal(shape).astype(np.float16)
    g = rng.normal(1, 0.1, (1, 16, 1, 1)).astype(np.float32)
    b = rng.normal(0, 0.1, (1, 16, 1, 1)).astype(np.float32)
    for _ in range(2):
        y, mean, var = bn(x, g, b)
        xf = x.astype(np.float32)
        np.testing.assert_allclose(mean.reshape(-1), xf.mean(axis=(0, 2, 3)), atol=1e-3)
        np.testing.assert_allclose(var.reshape(-1), xf.var(axis=(0, 2, 3)), atol=1e-3)
        want = (xf - xf.mean(axis=(0, 2, 3), keepdims=True)) / np.sqrt(xf.var(axis=(0, 2, 3), keepdims=True) + 1e-5) * g + b
        np.testing.assert_allclose(y.astype(np.float32), want, atol=1e-2, rtol=1e-2)


def test_scalar_parameters_and_argument_count():
    import dvm

    @dvm.kernel("vector", dynamic=True)
    def axpy(k, a, x, y):
        return k.store(k.add(k.mul(k.load(x, dvm.float32), k.scalar(a)), k.load(y, dvm.float32)))

    x = np.arange(1000, dtype=np.float32)
    y = np.ones(1000, np.float32)
    np.testing.assert_allclose(axpy(2.0, x, y), 2 * x + y, rtol=1e-6)
    np.testing.assert_allclose(axpy(-0.5, x, y), -0.5 * x + y, rtol=1e-6)
    with pytest.raises(TypeError):
        axpy(x, y)
