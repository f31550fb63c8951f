"""The variance pass folded into the mean pass (dvm_b200/csrc/stat_fusion.cc).

For a 16-bit tensor widened to fp32 the kernel does not run sum((x - mean)^2) as a pass of its own: the first pass takes
T = sum(x - s) and Q = sum((x - s)^2) for the first element s of each group, and the scalar code derives
sum(x) = T + n s and sum((x - m)^2) = Q - 2 (m - s) T + n (m - s)^2 from them.  Pinned here against the two-pass formula
in float64 at 1e-4 on well-conditioned data (the shapes of tests/ut/test_spec_vector.py:133-160 and
examples/02_batchnorm.py:19-60 of the reference), with the error bound spelled out on ill-conditioned data, and against
the unfolded three-pass kernel (DVM_B200_EXACT_MATH=1) of this library.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

import dvm_b200 as dvm
from dvm_b200 import workloads as W
from tests.util import assert_close, run_both

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _two_pass(x):
    xd = x.astype(np.float64)
    mean = xd.mean(axis=(0, 2, 3), keepdims=True)
    var = ((xd - mean) ** 2).mean(axis=(0, 2, 3), keepdims=True)
    return mean, var


def _bn(x, dtypes=None):
    n, c, hh, ww = x.shape
    gamma = np.ones((1, c, 1, 1), np.float32)
    beta = np.zeros((1, c, 1, 1), np.float32)
    dev, _, k = run_both(lambda kk, a, g, b: W.batchnorm_train(kk, a, g, b, n * hh * ww), [x, gamma, beta], dtypes=dtypes)
    assert " body_1:" in k.das() and " body_2:" not in k.das(), "the variance still has a pass of its own"
    return dev


def _bf16_round(a):
    u = a.astype(np.float32).view(np.uint32)
    u = (u + 0x7fff + ((u >> 16) & 1)) & 0xffff0000
    return u.view(np.float32)


@pytest.mark.parametrize("dt", ["fp16", "bf16"])
@pytest.mark.parametrize("shape", [(32, 64, 56, 56), (16, 32, 14, 14), (8, 3, 5, 7), (42, 5, 56, 56)])
def test_folded_variance_matches_the_two_pass_formula(shape, dt):
    rng = np.random.default_rng(21)
    x = (rng.normal(size=shape) * rng.uniform(0.5, 3.0, size=(1, shape[1], 1, 1)) + rng.normal(0, 2.0, size=(1, shape[1], 1, 1)))
    if dt == "bf16":
        x = _bf16_round(x)      # fp32 array holding bf16 values, uploaded as bf16 (dtype code 2)
        y, mean, var = _bn(x, dtypes=[2, None, None])
    else:
        x = x.astype(np.float16)
        y, mean, var = _bn(x)
    m64, v64 = _two_pass(x)
    assert np.max(np.abs(mean.astype(np.float64) - m64)) <= 1e-4 * (1.0 + np.max(np.abs(m64)))
    assert np.max(np.abs(var.astype(np.float64) - v64) / v64) <= 1e-4
    want = (x.astype(np.float64) - m64) / np.sqrt(v64 + 1e-5)
    assert_close(np.asarray(y).astype(np.float32), want.astype(np.float32), 2e-3 if dt == "fp16" else 1.6e-2, "normalised result")


def test_folded_variance_error_bound_on_ill_conditioned_channels():
    # a large offset, a first element far from the mean, a constant channel: the relative error of the variance stays
    # below 2e-6 * (1 + (mean - first)^2 / var), the bound the rewrite is applied under
    rng = np.random.default_rng(22)
    x = rng.normal(size=(16, 6, 28, 28)).astype(np.float32)
    x[:, 0] = x[:, 0] * 0.5 + 100.0            # offset 200 sigma: steps of 1/16 in fp16
    x[:, 1] = x[:, 1] * 4.0 - 1000.0           # offset, steps of 1/2
    x[0, 2, 0, 0] = 300.0                      # the reference value itself is an outlier
    x[0, 3, 0, 0] = -60000.0                   # ... by the full fp16 range
    x[:, 4] = 3.25                             # constant channel
    x = x.astype(np.float16)
    _, mean, var = _bn(x)
    m64, v64 = _two_pass(x)
    first = x[0:1, :, 0:1, 0:1].astype(np.float64)
    bound = 2e-6 * (1.0 + (m64 - first) ** 2 / np.maximum(v64, 1e-30))
    rel = np.abs(var.astype(np.float64) - v64) / np.maximum(v64, 1e-30)
    for c in (0, 1, 2, 3, 5):
        assert rel[0, c, 0, 0] <= max(bound[0, c, 0, 0], 1e-5), (c, rel[0, c, 0, 0], bound[0, c, 0, 0])
    assert abs(float(var[0, 4, 0, 0])) <= 1e-9 and abs(float(mean[0, 4, 0, 0]) - 3.25) <= 1e-6
    # the mean comes from T + n s: its error follows the distance between the reference value and the mean
    assert np.all(np.abs(mean.astype(np.float64) - m64) <= 1e-6 + 2e-7 * (np.abs(m64) + np.abs(m64 - first)))


def test_folded_and_unfolded_kernels_agree(tmp_path):
    # the same graph through the three-pass kernel (DVM_B200_EXACT_MATH=1) in a child process
    code = ("import sys, numpy as np, dvm_b200 as dvm\n"
            "from dvm_b200 import workloads as W\n"
            "from tests.util import run_both\n"
            "x = np.load(sys.argv[1])\n"
            "n, c, hh, ww = x.shape\n"
            "g = np.ones((1, c, 1, 1), np.float32); b = np.zeros((1, c, 1, 1), np.float32)\n"
            "dev, _, k = run_both(lambda kk, a, gg, bb: W.batchnorm_train(kk, a, gg, bb, n * hh * ww), [x, g, b])\n"
            "assert ' body_2:' in k.das()\n"
            "np.savez(sys.argv[2], y=dev[0], mean=dev[1], var=dev[2])\n")
    rng = np.random.default_rng(23)
    x = (rng.normal(size=(24, 16, 28, 28)) * 1.7 + 0.4).astype(np.float16)
    np.save(tmp_path / "x.npy", x)
    env = dict(os.environ, PYTHONPATH=ROOT, DVM_B200_EXACT_MATH="1")
    subprocess.run([sys.executable, "-c", code, str(tmp_path / "x.npy"), str(tmp_path / "out.npz")], env=env, check=True, cwd=ROOT)
    exact = np.load(tmp_path / "out.npz")
    y, mean, var = _bn(x)
    assert_close(mean, exact["mean"], 1e-5, "mean")
    assert_close(var, exact["var"], 1e-5, "var")
    # the normalised fp16 result may differ by one unit in the last place where the fp32 value sits on a rounding edge
    diff = np.abs(y.astype(np.float32) - exact["y"].astype(np.float32))
    assert np.max(diff) <= 2e-3 and np.mean(diff > 0) < 0.01


@pytest.mark.parametrize("shape,dims", [((64, 4096), (1,)), ((300, 777), (1,)), ((37, 5000), (1,)), ((48, 96, 64), (2,)),
                                        ((48, 96, 64), (1, 2)), ((96, 64, 50), (0,)), ((7, 33), (0, 1)), ((2048, 16), (1,))])
def test_folded_variance_over_other_axes(shape, dims):
    # layer-norm style statistics (rows, trailing blocks, leading axis, everything): the same rewrite on every geometry
    rng = np.random.default_rng(24)
    x = (rng.normal(size=shape) * 1.5 + rng.normal(0, 2.0, size=[s if i not in dims else 1 for i, s in enumerate(shape)])).astype(np.float16)
    n = int(np.prod([shape[d] for d in dims]))

    def build(k, a):
        xf = k.cast(a, 3)
        mean = k.mul(k.sum(xf, dims, True), 1.0 / n)
        xc = k.sub(xf, mean)
        var = k.mul(k.sum(k.mul(xc, xc), dims, True), 1.0 / n)
        y = k.cast(k.div(xc, k.sqrt(k.add(var, 1e-5))), 1)
        return y, mean, var

    dev, _, k = run_both(build, [x])
    assert " body_1:" in k.das() and " body_2:" not in k.das()
    xd = x.astype(np.float64)
    m64 = xd.mean(axis=dims, keepdims=True)
    v64 = ((xd - m64) ** 2).mean(axis=dims, keepdims=True)
    assert np.max(np.abs(dev[1].astype(np.float64) - m64)) <= 1e-4 * (1.0 + np.max(np.abs(m64)))
    assert np.max(np.abs(dev[2].astype(np.float64) - v64) / np.maximum(v64, 1e-12)) <= 2e-4
    assert_close(np.asarray(dev[0]).astype(np.float32), ((xd - m64) / np.sqrt(v64 + 1e-5)).astype(np.float32), 2e-3, "normalised")
