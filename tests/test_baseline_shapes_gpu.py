"""Device parity at the benchmark's own shapes for the three vector-path graphs: the fused elementwise chain on
fp32 [8192, 8192], the BatchNorm training-forward graph on fp16 [64, 256, 56, 56] and the residual + RMSNorm +
SwiGLU graph on bf16 [T, 4096] at T = 1000, 4096, 16384.

The kernels are built exactly as ``bench.py`` builds the ones it times (``bench.DeviceWorkload``: same graph
definition, kernel type, seeded inputs), so the launch geometry picked from the shape -- grid, chunk size, ring
depth, kernel variant -- is the geometry the reported numbers come from; the test asserts the geometry line of
the listing as well.  Every element of every output is compared with the NumPy oracle under the class tolerances
(1e-5 fp32 elementwise, 1e-2 for 16-bit storage and reductions), and the statistics additionally with NumPy's
own mean / var.  Graph formulas: examples/01_add.py:19-25, examples/02_batchnorm.py:19-60,
tests/ut/test_spec_vector.py:133-160 of the reference.
"""
import re

import numpy as np
import pytest

import bench
from tests.util import TOL_FP32, TOL_HALF, TOL_REDUCE, as_f32, assert_close

pytestmark = pytest.mark.gpu


def _geometry(das):
    """The fields of the `vmain.sm100(...)` line of a listing as a dict of strings."""
    m = re.search(r"vmain\.sm100\(([^)]*)\)", das)
    assert m, das[:200]
    out = {}
    for part in m.group(1).split(", "):
        key, _, val = part.partition("=")
        out[key.strip()] = val.strip()
    return out


def _run(name, scale=1.0):
    wl = bench.DeviceWorkload(name, scale=scale)
    das = wl.k.das()
    assert das.count("vmain") == 1 and "mmain" not in das, "the graph must be one launch of the vector interpreter"
    wl.k.run()
    dev = wl.outputs()
    ref = bench.cpu_eval(name, wl.arrays)
    arrays = wl.arrays
    wl.k.release_io()
    return dev, ref, arrays, _geometry(das)


def _checksum(a):
    return float(as_f32(a).astype(np.float64).sum())


def test_c1_fused_elementwise_full_size():
    dev, ref, arrays, geo = _run("c1")
    assert dev[0].shape == (8192, 8192)
    assert geo["mode"] == "flat" and geo["groups"] == "1" and geo["group_elems"] == str(8192 * 8192)
    assert int(geo["grid"]) % 148 == 0
    assert_close(dev[0], ref[0], TOL_FP32, "c1 full size")
    x, y = arrays
    assert_close(dev[0], np.exp(x) * y + np.float32(0.5), TOL_FP32, "c1 against the plain formula")
    assert abs(_checksum(dev[0]) - _checksum(ref[0])) <= 1e-6 * np.abs(as_f32(ref[0])).astype(np.float64).sum()


def test_c2_batchnorm_full_size():
    dev, ref, arrays, geo = _run("c2")
    x = arrays[0]
    assert dev[0].shape == (64, 256, 56, 56) and dev[0].dtype == np.float16
    assert geo["mode"] == "group" and geo["groups"] == "256" and geo["group_elems"] == str(64 * 56 * 56)
    assert_close(dev[0], ref[0], TOL_HALF, "c2 y")
    assert_close(dev[1], ref[1], TOL_REDUCE, "c2 mean")
    assert_close(dev[2], ref[2], TOL_REDUCE, "c2 var")
    # the statistics far inside their class: fp32 tree sums against NumPy's pairwise sums of 200704 values
    xf = x.astype(np.float32)
    mean = xf.mean(axis=(0, 2, 3), dtype=np.float64)
    var = xf.var(axis=(0, 2, 3), dtype=np.float64)
    assert_close(dev[1].reshape(-1), mean.astype(np.float32), 1e-4, "c2 mean against numpy")
    assert_close(dev[2].reshape(-1), var.astype(np.float32), 1e-4, "c2 var against numpy")
    # y is normalised: per channel mean beta and variance gamma^2 (size-independent property of the whole output)
    yf = dev[0].astype(np.float32)
    gamma, beta = arrays[1].reshape(-1), arrays[2].reshape(-1)
    assert_close(yf.mean(axis=(0, 2, 3), dtype=np.float64).astype(np.float32), beta, 2e-3, "c2 mean of y")
    assert_close(yf.std(axis=(0, 2, 3), dtype=np.float64).astype(np.float32), np.abs(gamma), 2e-3, "c2 std of y")


@pytest.mark.parametrize("tokens", [1000, 4096, 16384])
def test_c3_rmsnorm_swiglu_at_benchmark_token_counts(tokens):
    dev, ref, arrays, geo = _run("c3", scale=tokens / 16384.0)
    assert dev[0].shape == (tokens, 4096) and dev[1].shape == (tokens, 4096)
    assert geo["mode"] == "group" and geo["groups"] == str(tokens) and geo["group_elems"] == "4096"
    assert_close(dev[0], ref[0], TOL_HALF, "c3 rmsnorm(h + r) * w at T=%d" % tokens)
    assert_close(dev[1], ref[1], TOL_HALF, "c3 silu(g) * u at T=%d" % tokens)
    # the plain formulas on every row
    h, r, w, g, u = (as_f32(a) for a in arrays)
    s = h + r
    want1 = s / np.sqrt((s * s).mean(axis=1, keepdims=True) + 1e-6) * w
    want2 = g / (1.0 + np.exp(-g)) * u
    assert_close(dev[0], want1, TOL_HALF, "c3 out1 against numpy")
    assert_close(dev[1], want2, TOL_HALF, "c3 out2 against numpy")
    for d, o in zip(dev, ref):
        scale = np.abs(as_f32(o)).astype(np.float64).sum()
        assert abs(_checksum(d) - _checksum(o)) <= 1e-4 * scale
