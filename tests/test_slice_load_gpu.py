"""Kernel::SliceLoad / StridedSliceLoad (include/dvm.h:305-317) on the device: a window of a tensor in memory read as a
strided load.  Cases follow the reference's tests/ut/test_slice.py (1-d, 2-d and 3-d windows by start + size, windows by
start / end / step with negative and out-of-range indices, a window that broadcasts against another tensor)."""
import numpy as np
import pytest

from dvm_b200.tester import Tester
from tests.util import TOL_FP32, TOL_HALF, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("shape,start,size", [((32,), (3,), (16,)), ((1111,), (222,), (333,)), ((1621,), (4,), (333,)),
                                              ((32, 32), (3, 3), (16, 16)), ((4, 4097), (0, 5), (2, 4000)),
                                              ((32, 32, 4), (3, 3, 1), (16, 16, 2)), ((32, 32, 10), (3, 3, 1), (8, 13, 8)),
                                              ((4, 4097, 20), (0, 0, 5), (2, 4097, 5)), ((111, 111, 111), (22, 22, 22), (33, 33, 32))])
def test_window_by_start_and_size(dtype, shape, start, size):
    rng = np.random.default_rng(41)
    a = rng.normal(0, 1, shape).astype(dtype)
    t = Tester("vector")
    s = t.store(t.mul(t.slice_load(a, start, size), 2))
    t.run()
    want = 2 * a[tuple(slice(b, b + n) for b, n in zip(start, size))].astype(np.float32)
    assert_close(np.asarray(t.output(s)).astype(np.float32), want, TOL_FP32 if dtype == np.float32 else TOL_HALF, "slice load")
    assert "workspace_bytes=0" in t.inspect()          # the window is read in place


@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.int32])
@pytest.mark.parametrize("shape,start,end", [((32, 32, 4), 1, -2), ((32, 7, 7), -30, 12), ((32, 7, 7), -30, 100),
                                             ((14, 4097, 20), -4, -1)])
def test_window_by_start_and_end_as_python_slices(dtype, shape, start, end):
    rng = np.random.default_rng(42)
    a = (rng.normal(0, 1, shape) * (10 if dtype == np.int32 else 1)).astype(dtype)
    t = Tester("vector")
    x = t.stridedslice_load(a, (start, 0, 0), (end, shape[1], shape[2]), (1, 1, 1))
    s = t.store(t.mul(x, 2))
    t.run()
    want = 2 * a[start:end]
    got = np.asarray(t.output(s))
    if dtype == np.int32:
        assert np.array_equal(got, want)
    else:
        assert_close(got.astype(np.float32), want.astype(np.float32), TOL_FP32 if dtype == np.float32 else TOL_HALF, "strided slice load")


def test_steps_and_a_window_that_broadcasts():
    rng = np.random.default_rng(43)
    a = rng.normal(0, 1, [40, 60]).astype(np.float32)
    t = Tester("vector")
    s0 = t.store(t.add(t.stridedslice_load(a, (1, 2), (39, 60), (3, 2)), 1.0))
    t.run()
    assert_close(t.output(s0), a[1:39:3, 2:60:2] + np.float32(1.0), TOL_FP32, "steps 3 and 2")
    a4 = rng.normal(0, 1, [1, 10, 20, 30]).astype(np.float32)
    b4 = rng.normal(0, 1, [10, 10, 20, 1]).astype(np.float32)
    t = Tester("vector")
    x = t.slice_load(a4, (0, 2, 4, 6), (1, 5, 10, 20))
    y = t.slice_load(b4, (1, 2, 4, 0), (8, 5, 10, 1))
    s1 = t.store(t.add(x, y))
    t.run()
    assert_close(t.output(s1), a4[:, 2:7, 4:14, 6:26] + b4[1:9, 2:7, 4:14, :], TOL_FP32, "two windows, broadcast")
