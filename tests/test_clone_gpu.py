"""Kernel::Clone on the device (include/dvm.h:255-259; RtKernelPy::Clone, src/pybind_api.cc:918-997): a kernel built once
and copied runs on its own inputs.  Cases follow the reference's tests/ut/test_clone.py (static and dynamic vector
kernels, a speculative one, a MatMul with post-fusion)."""
import numpy as np
import pytest

from dvm_b200.tester import Tester
from tests.util import TOL_HALF, assert_close

pytestmark = pytest.mark.gpu


def test_static_vector_kernel_and_its_copy():
    rng = np.random.default_rng(61)
    a = rng.normal(0, 1, [10, 512]).astype(np.float32)
    t = Tester("vector")
    ax = t.load(a)
    out = t.store(t.sum(t.add(ax, 0.01), [0], True))
    t.run()
    assert_close(t.output(out), np.sum(a + np.float32(0.01), (0,), keepdims=True), 1e-4, "base kernel")
    t2 = Tester("vector")
    ax2, out2 = t2.clone(t, [ax, out])
    a2 = rng.normal(0, 1, [10, 512]).astype(np.float32)
    t2.input(ax2, a2)
    t2.run()
    assert_close(t2.output(out2), np.sum(a2 + np.float32(0.01), (0,), keepdims=True), 1e-4, "copy on its own input")
    assert_close(t.output(out), np.sum(a + np.float32(0.01), (0,), keepdims=True), 1e-4, "base untouched")


def test_dynamic_kernel_copy_with_its_own_shape_and_reduce_dims():
    rng = np.random.default_rng(62)
    t = Tester("vector:dyn")
    ax = t.load([], "float32")
    dims = t.int_array()
    out = t.store(t.sum(t.add(ax, 0.01), dims, True))
    a = rng.normal(0, 1, [10, 512]).astype(np.float32)
    t.input(ax, a)
    dims.update([0])
    t.run()
    assert_close(t.output(out), np.sum(a + np.float32(0.01), (0,), keepdims=True), 1e-4, "base kernel")
    t2 = Tester("vector:dyn")
    ax2, out2, dims2 = t2.clone(t, [ax, out, dims])
    a2 = rng.normal(0, 1, [64, 800]).astype(np.float32)
    t2.input(ax2, a2)
    dims2.update([1])
    t2.run()
    assert_close(t2.output(out2), np.sum(a2 + np.float32(0.01), (1,), keepdims=True), 1e-4, "copy, other shape and dims")


def test_matmul_with_post_fusion_and_its_copy():
    rng = np.random.default_rng(63)

    def data():
        return (rng.normal(0, 0.5, [128, 64]).astype(np.float16), rng.normal(0, 0.5, [64, 256]).astype(np.float16))

    a, b = data()
    t = Tester("mix")
    la, lb = t.load(a), t.load(b)
    out = t.store(t.add(t.matmul(la, lb, False, False), 1.0))
    t.run()
    want = lambda x, y: (x.astype(np.float32) @ y.astype(np.float32)).astype(np.float16).astype(np.float32) + 1.0
    assert_close(np.asarray(t.output(out)).astype(np.float32), want(a, b), TOL_HALF, "base kernel")
    t2 = Tester("mix")
    la2, lb2, out2 = t2.clone(t, [la, lb, out])
    a2, b2 = data()
    t2.input(la2, a2)
    t2.input(lb2, b2)
    t2.run()
    assert_close(np.asarray(t2.output(out2)).astype(np.float32), want(a2, b2), TOL_HALF, "copy")
