"""Strided (view) loads and stores on the device: Kernel::Load(addr, shape, stride, type) / Store(addr, input, stride)
(include/dvm.h:286-294, 332-339).  Cases follow the reference's tests/ut/test_view.py (2-d and 3-d windows of a larger
array, a strided store into a zero-filled buffer), plus the channel slab of an NCHW tensor that the BatchNorm graph
is partitioned by, an element offset into the source array, and a view that feeds a MatMul (copied out first)."""
import numpy as np
import pytest

from dvm_b200 import workloads as W
from dvm_b200.tester import Tester
from tests.util import TOL_FP32, TOL_HALF, TOL_REDUCE, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("in_shape,window", [([30, 1000], [20, 500]), ([30, 500], [20, 200]), ([30, 4000], [20, 3000]),
                                             ([43, 1000], [40, 500]), ([7, 13], [5, 11])])
def test_window_of_a_matrix(in_shape, window):
    rng = np.random.default_rng(1)
    a = rng.normal(0, 1, in_shape).astype(np.float32)
    t = Tester("vector")
    x = t.view_load(window, [in_shape[1], 1], a)
    s = t.store(t.add(x, 0.1))
    t.run()
    assert_close(t.output(s), a[:window[0], :window[1]] + np.float32(0.1), TOL_FP32, "2-d window")


@pytest.mark.parametrize("in_shape,window", [([24, 20, 100], [20, 10, 60]), ([24, 20, 1000], [20, 10, 600]),
                                             ([24, 20, 1000], [20, 20, 600]), ([24, 20, 64], [20, 15, 64]),
                                             ([200, 20, 100], [200, 20, 30]), ([200, 20, 20], [200, 10, 20])])
def test_window_of_a_3d_tensor(in_shape, window):
    rng = np.random.default_rng(2)
    a = rng.normal(0, 1, in_shape).astype(np.float32)
    t = Tester("vector")
    x = t.view_load(window, [in_shape[1] * in_shape[2], in_shape[2], 1], a)
    s = t.store(t.add(x, 0.1))
    t.run()
    assert_close(t.output(s), a[:window[0], :window[1], :window[2]] + np.float32(0.1), TOL_FP32, "3-d window")


def test_strided_store_leaves_the_rest_of_the_buffer_alone():
    rng = np.random.default_rng(3)
    data = rng.normal(0, 0.2, (4, 96, 7, 7)).astype(np.float32)
    stride = [96 * 49, 49, 7, 1]
    t = Tester("vector")
    x = t.view_load([4, 32, 7, 7], stride, data)
    expected = np.zeros_like(data)
    expected[:, :32] = data[:, :32]
    t.view_store_expect(x, stride, expected)
    assert t.run_check()


def test_element_offset_and_transposed_view():
    rng = np.random.default_rng(4)
    a = rng.normal(0, 1, (64, 48)).astype(np.float32)
    t = Tester("vector")
    x = t.view_load([40, 16], [48, 1], a, offset=3 * 48 + 5)   # rows 3.., columns 5..20
    y = t.view_load([48, 64], [1, 48], a)                       # the transpose, read through its strides
    s1, s2 = t.store(t.mul(x, 2.0)), t.store(t.sum(y, (1,), True))
    t.run()
    assert_close(t.output(s1), a[3:43, 5:21] * 2, TOL_FP32, "offset window")
    assert_close(t.output(s2), a.T.sum(axis=1, keepdims=True), 1e-4, "row sums of the transposed view")


@pytest.mark.parametrize("first,count", [(0, 8), (24, 8), (5, 3)])
def test_batchnorm_on_a_channel_slab_of_nchw(first, count):
    """The partitioning of the BatchNorm graph over GPUs: a rank normalises channels [first, first + count) of an NCHW
    tensor in place in the full-size buffers, through strided loads and stores."""
    rng = np.random.default_rng(5)
    n, c, h, w = 16, 32, 14, 14
    x = rng.normal(size=(n, c, h, w)).astype(np.float16)
    gamma = rng.normal(1, 0.1, (1, c, 1, 1)).astype(np.float32)
    beta = rng.normal(0, 0.1, (1, c, 1, 1)).astype(np.float32)
    stride = [c * h * w, h * w, w, 1]
    t = Tester("vector")
    xs = t.view_load([n, count, h, w], stride, x, offset=first * h * w)
    g, b = t.load(gamma[:, first:first + count]), t.load(beta[:, first:first + count])
    y, mean, var = W.batchnorm_train(t, xs, g, b, n * h * w)
    ys = t.view_store(y, stride)
    t.set_output(ys, np.zeros_like(x), offset=first * h * w)   # the slab starts `first` channels into the result
    sm, sv = t.store(mean), t.store(var)
    t.run()
    xf = x[:, first:first + count].astype(np.float32)
    m, v = xf.mean(axis=(0, 2, 3), keepdims=True), xf.var(axis=(0, 2, 3), keepdims=True)
    want = (xf - m) / np.sqrt(v + 1e-5) * gamma[:, first:first + count] + beta[:, first:first + count]
    got = t.output(ys)
    assert_close(got[:, first:first + count], want, TOL_HALF, "normalised slab")
    outside = got.copy()
    outside[:, first:first + count] = 0
    assert not outside.any(), "elements outside the slab were written"
    assert_close(t.output(sm), m, TOL_REDUCE, "slab mean")
    assert_close(t.output(sv), v, TOL_REDUCE, "slab variance")


def test_view_feeding_a_matmul_is_copied_out_first():
    rng = np.random.default_rng(6)
    big = rng.normal(0, 0.1, (256, 512)).astype(np.float32)
    b = rng.normal(0, 0.1, (128, 192)).astype(np.float32)
    t = Tester("split")
    a = t.view_load([256, 128], [512, 1], big.astype(np.float16))
    s = t.store(t.matmul(a, t.load(b.astype(np.float16)), False, False))
    t.run()
    assert t.das().count("vmain") == 1 and t.das().count("mmain") == 1
    want = big[:, :128].astype(np.float16).astype(np.float32) @ b.astype(np.float16).astype(np.float32)
    assert_close(t.output(s), want, TOL_HALF, "MatMul of a window")


def test_permute_slice_and_split_of_a_tensor_in_memory():
    """Kernel::Permute / Slice / Split (include/dvm.h:428-453, 470-479) of a Load: pure views, no copy."""
    rng = np.random.default_rng(7)
    a = rng.normal(size=(6, 40, 96)).astype(np.float32)
    t = Tester("vector")
    x = t.load(a)
    p = t.permute(x, [2, 0, 1])
    s1 = t.store(t.add(p, 1.0))
    s2 = t.store(t.mul(t.slice(x, [1, 8, 16], [4, 20, 64]), 2.0))
    s3 = t.store(t.sum(t.slice_dim(x, 1, -10, 40), (2,), True))
    chunks = t.split(x, 2, 40, 3)                       # 40 + 40 + 16 columns
    s4 = [t.store(t.mul(c, 3.0)) for c in chunks]
    t.run()
    assert_close(t.output(s1), a.transpose(2, 0, 1) + 1.0, TOL_FP32, "permute")
    assert_close(t.output(s2), a[1:5, 8:28, 16:80] * 2.0, TOL_FP32, "slice")
    assert_close(t.output(s3), a[:, 30:40].sum(axis=2, keepdims=True), 1e-4, "slice along one dim")
    for i, s in enumerate(s4):
        assert_close(t.output(s), a[:, :, 40 * i:40 * (i + 1)] * 3.0, TOL_FP32, "split chunk %d" % i)


def test_views_of_computed_values_and_of_views():
    rng = np.random.default_rng(8)
    a = rng.normal(size=(64, 128)).astype(np.float32)
    b = rng.normal(size=(128, 64)).astype(np.float32)
    t = Tester("split")
    y = t.add(t.load(a), 1.0)                            # computed: written to the workspace, then viewed
    yt = t.permute(y, [1, 0])
    s1 = t.store(t.mul(yt, t.load(b)))
    s2 = t.store(t.exp(t.slice(yt, [16, 8], [32, 40])))  # a view of a view
    t.run()
    want = (a + 1.0).T
    assert_close(t.output(s1), want * b, TOL_FP32, "permute of a computed value")
    assert_close(t.output(s2), np.exp(want[16:48, 8:48]), TOL_FP32, "slice of a permuted value")


def _dense_strides(shape):
    st = [1] * len(shape)
    for i in range(len(shape) - 1, 0, -1):
        st[i - 1] = st[i] * shape[i]
    return st


@pytest.mark.parametrize("in_shape,window", [([4, 4, 5, 3, 16], [3, 2, 3, 2, 12]), ([4, 4, 4, 5, 6, 16], [3, 2, 3, 4, 5, 12])])
def test_windows_of_five_and_six_dimensions(in_shape, window):
    # more strided axes than a tile walks: the outer ones become the launch's groups (tests/ut/test_view.py:92-114)
    rng = np.random.default_rng(51)
    a = rng.normal(0, 1, in_shape).astype(np.float32)
    t = Tester("vector")
    s = t.store(t.add(t.view_load(window, _dense_strides(in_shape), a), 0.1))
    t.run()
    assert_close(t.output(s), a[tuple(slice(0, w) for w in window)] + np.float32(0.1), TOL_FP32, "%d-d window" % len(window))
    assert "mode=group" in t.das()


def test_high_rank_window_that_broadcasts_against_a_dense_tensor():
    # tests/ut/test_view.py:217-233
    rng = np.random.default_rng(52)
    shape, sshape, bshape = [1, 10, 1, 20, 8, 32], [1, 6, 1, 18, 7, 32], [4, 6, 8, 18, 7, 32]
    a = rng.normal(0, 1, shape).astype(np.float32)
    b = rng.normal(0, 1, bshape).astype(np.float32)
    t = Tester("vector")
    s = t.store(t.add(t.view_load(sshape, _dense_strides(shape), a), t.load(b)))
    t.run()
    assert_close(t.output(s), a[:, :6, :, :18, :7, :] + b, TOL_FP32, "6-d window + dense tensor")


def test_strided_store_of_five_dimensions():
    # tests/ut/test_view.py:364-375
    rng = np.random.default_rng(53)
    out_shape, window = [4, 4, 5, 3, 16], [3, 2, 3, 2, 12]
    a = rng.normal(0, 1, window).astype(np.float32)
    t = Tester("vector")
    want = np.zeros(out_shape, np.float32)
    want[tuple(slice(0, w) for w in window)] = a + np.float32(0.1)
    t.view_store_expect(t.add(t.load(a), 0.1), _dense_strides(out_shape), want)
    assert t.run_check()


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
@pytest.mark.parametrize("shape,pad", [((200, 100), 128), ((220, 100), 202), ((2000, 1), 1), ((1, 3, 200, 100), 128),
                                       ((4, 5, 111, 1), 1), ((1024, 30), 15), ((7, 33), 0)])
def test_pad_store_writes_rows_into_a_wider_buffer(dtype, shape, pad):
    # Kernel::PadStore (include/dvm.h:344): the store's shape is the buffer's, rows longer by the pad, the padding untouched
    # (tests/ut/test_pad.py)
    rng = np.random.default_rng(71)
    a = rng.normal(0, 1, shape).astype(dtype)
    t = Tester("vector")
    o = t.pad_store(t.abs(t.load(a)), pad)
    t.run()
    out = np.asarray(t.output(o))
    assert out.shape == tuple(shape[:-1]) + (shape[-1] + pad,)
    assert_close(out[..., :shape[-1]].astype(np.float32), np.abs(a).astype(np.float32), 0.0, "pad store")
