"""Kernel::Concat (include/dvm.h:455-469) on the device.  Cases follow the reference's tests/ut/test_view_sch.py:111-160
(three inputs, two of them computed, along the inner, a middle and the outer dimension, followed by an add with or
without a broadcast; one input that holds almost all elements beside many small ones) and test_elemwise.py's
concatenation of loads; results are compared with numpy.concatenate."""
import numpy as np
import pytest

from dvm_b200.tester import Tester
from tests.util import TOL_FP32, TOL_HALF, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("shape1,shape2,shape3,shape4,axis", [
    ([3, 400], [3, 600], [3, 200], [3, 1200], 1),                       # inner
    ([3, 400], [3, 600], [3, 200], [3, 1], 1),                          # inner, the add broadcasts
    ([3, 400, 32], [3, 600, 32], [3, 200, 32], [3, 1200, 32], 1),       # middle
    ([3, 400, 32], [3, 600, 32], [3, 200, 32], [3, 1, 32], 1),          # middle, the add broadcasts
    ([10, 400], [20, 400], [30, 400], [60, 400], 0),                    # outer
    ([10, 400], [20, 400], [30, 400], [60, 1], 0),                      # outer, the add broadcasts
    ([5, 7], [5, 9], [5, 1], [5, 17], -1),                              # small and ragged, negative dimension
])
def test_concat_of_computed_values_and_loads(dtype, shape1, shape2, shape3, shape4, axis):
    rng = np.random.default_rng(31)
    a0, a1, a2, a3 = (rng.normal(0, 1, s).astype(dtype) for s in (shape1, shape2, shape3, shape4))
    t = Tester("vector")
    x2 = t.add(t.load(a0), 0.1)
    x3 = t.mul(t.load(a1), 0.6)
    x5 = t.concat([x2, x3, t.load(a2)], axis)
    s = t.store(t.add(x5, t.load(a3)))
    t.run()
    f = np.float32
    want = np.concatenate([a0.astype(f) + f(0.1), a1.astype(f) * f(0.6), a2.astype(f)], axis=axis) + a3.astype(f)
    if dtype == np.float16:   # each op rounds to fp16, as the kernel's ops do
        want = (np.concatenate([(a0 + dtype(0.1)).astype(dtype), (a1 * dtype(0.6)).astype(dtype), a2], axis=axis) + a3).astype(f)
    assert_close(np.asarray(t.output(s)).astype(f), want, TOL_FP32 if dtype == np.float32 else TOL_HALF, "concat + add")
    assert t.das().count("vmain.") >= 4          # one launch per slab, one for the ops behind the result


def test_one_large_and_many_small_inputs():
    rng = np.random.default_rng(32)
    t = Tester("vector")
    first = rng.normal(0, 1, [137862, 32]).astype(np.float32)
    parts, ops = [first + np.float32(0.1)], [t.add(t.load(first), 0.1)]
    for _ in range(20):
        a = rng.normal(0, 1, [2, 32]).astype(np.float32)
        parts.append(a + np.float32(0.1))
        ops.append(t.add(t.load(a), 0.1))
    s = t.store(t.mul(t.concat(ops, 0), 0.5))
    t.run()
    assert_close(t.output(s), np.concatenate(parts, axis=0) * np.float32(0.5), TOL_FP32, "concat of 21 inputs")


def test_concat_result_stored_directly_and_used_twice():
    rng = np.random.default_rng(33)
    a, b = rng.normal(0, 1, [64, 96]).astype(np.float32), rng.normal(0, 1, [64, 32]).astype(np.float32)
    t = Tester("vector")
    cat = t.concat([t.load(a), t.load(b)], 1)
    s0 = t.store(cat)
    s1 = t.store(t.sum(t.mul(cat, cat), (1,), True))
    t.run()
    want = np.concatenate([a, b], axis=1)
    assert_close(t.output(s0), want, 0.0, "the concatenation itself")
    assert_close(t.output(s1), (want * want).sum(axis=1, keepdims=True), 1e-4, "a row reduction over it")
