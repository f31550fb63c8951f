"""Pins the CPU oracle to the expectations the reference's own tests compute.

The reference stores no golden vectors: each of its tests builds a graph and compares the device result with a NumPy
formula under a stated tolerance.  Each case here evaluates the same graph with the oracle and checks it against the
same NumPy formula under the same tolerance, citing the reference test it restates.  The committed fixtures in
tests/golden/ (made by tests/golden/make_golden.py) freeze the oracle's outputs so that a later change to the oracle
is noticed.  Runs on CPU.
"""
import os

import numpy as np
import pytest

from dvm_b200 import workloads as W
from oracle.dvm_oracle import BF16, BOOL, F16, F32, I32, OracleKernel

HERE = os.path.dirname(os.path.abspath(__file__))


def close(got, want, eps):
    got = np.asarray(got).astype(np.float64) if np.asarray(got).dtype.kind in "fb" or str(np.asarray(got).dtype) == "bfloat16" else np.asarray(got)
    return np.allclose(got, np.asarray(want).astype(got.dtype), rtol=eps, atol=eps, equal_nan=True)


@pytest.mark.parametrize("dt,eps", [(np.float16, 1e-3), (np.float32, 1e-5)])
def test_gelu_expander_8_op(dt, eps):
    # tests/ut/test_composite_ops.py:25-26, 53-71
    np.random.seed(12)
    a = np.random.normal(0, 1, [32, 1024]).astype(dt)
    o = OracleKernel()
    got = o.store(W.gelu_tanh(o, o.load(a)))
    want = 0.5 * a * (1 + np.tanh(np.sqrt(2 / np.pi) * (a + 0.044715 * np.power(a, 3))))
    assert close(got, want, eps if dt == np.float32 else 2e-3)


@pytest.mark.parametrize("dt,eps", [(np.float16, 1e-3), (np.float32, 1e-5)])
def test_tanh_through_exp(dt, eps):
    # tests/ut/test_composite_ops.py:29-50
    a = np.random.default_rng(0).normal(0, 1, [32, 1024]).astype(dt)
    o = OracleKernel()
    x = o.load(a)
    e, fe = o.exp(x), o.exp(o.mul(x, -1.0))
    got = o.store(o.div(o.sub(e, fe), o.add(e, fe)))
    assert close(got, np.tanh(a), eps if dt == np.float32 else 2e-3)


def test_rmsnorm_fp16():
    # tests/ut/test_spec_vector.py:133-160 (tolerance 3e-3)
    rng = np.random.default_rng(17)
    for rows, cols in [(2, 8192), (17, 129)]:
        x_data = rng.normal(0, 1, (rows, cols)).astype(np.float16)
        gamma = rng.normal(1, 0.1, (cols,)).astype(np.float16)
        o = OracleKernel()
        x = o.cast(o.load(x_data), F32)
        ss = o.sum(o.mul(x, x), [1], True)
        rstd = o.div(1.0, o.sqrt(o.add(o.div(ss, float(cols)), 1e-6)))
        got = o.store(o.mul(o.cast(o.mul(x, rstd), F16), o.load(gamma)))
        xr = x_data.astype(np.float32)
        want = (xr * (1.0 / np.sqrt(np.mean(xr * xr, axis=1, keepdims=True) + 1e-6))).astype(np.float16) * gamma
        assert close(got, want, 3e-3)


@pytest.mark.parametrize("t1,t2,eps", [(np.float16, np.float32, 1e-3), (np.float32, np.float16, 1e-3), (np.float16, np.int32, 0),
                                       (np.int32, np.float32, 1e-5), (np.int32, np.float16, 1e-3)])
def test_cast(t1, t2, eps):
    # tests/ut/test_cast.py:25-36 (float -> int truncates toward zero, eps 0)
    a = np.random.default_rng(1).normal(0, 100, [1024, 32]).astype(t1)
    o = OracleKernel()
    to = {np.float16: F16, np.float32: F32, np.int32: I32}[t2]
    got = o.store(o.copy(o.cast(o.copy(o.load(a)), to)))
    with np.errstate(over="ignore"):
        want = a.astype(t2)
    assert got.dtype == np.dtype(t2)
    assert close(got, want, eps)


def test_cast_bf16_round_trip():
    # tests/ut/test_cast.py:39-49 (eps 1e-2)
    a = np.random.default_rng(2).normal(0, 100, [1024, 32]).astype(np.float32)
    o = OracleKernel()
    got = o.store(o.cast(o.load(a, BF16), F32))
    assert close(got, a, 1e-2)
    got = o.store(o.cast(o.load(a), BF16)).astype(np.float32)
    assert close(got, a, 1e-2)


def test_cast_to_bool_with_special_values():
    # tests/ut/test_cast.py:151-165: x != 0, so NaN and infinities are true, -0.0 is false
    a = np.array([0.0, -0.0, 1.5, np.nan, np.inf, -np.inf, 1e-30], dtype=np.float32)
    o = OracleKernel()
    got = o.store(o.cast(o.load(a), BOOL))
    assert got.dtype == np.bool_ and (got == (a != 0)).all()


def test_compare_with_nan_and_select():
    # tests/ut/test_cmp.py:24-120, tests/ut/test_select.py:27-64
    a = np.array([1.0, np.nan, 3.0, -1.0], dtype=np.float32)
    b = np.array([1.0, 2.0, np.nan, -2.0], dtype=np.float32)
    o = OracleKernel()
    x, y = o.load(a), o.load(b)
    for name, fn in [("equal", np.equal), ("not_equal", np.not_equal), ("greater", np.greater),
                     ("greater_equal", np.greater_equal), ("less", np.less), ("less_equal", np.less_equal)]:
        got = o.store(getattr(o, name)(x, y))
        assert got.dtype == np.bool_ and (got == fn(a, b)).all(), name
    got = o.store(o.select(o.greater(x, y), x, y))
    assert close(got, np.where(a > b, a, b), 0)


@pytest.mark.parametrize("shape,dims,keep", [((64, 300), (1,), True), ((5, 7, 64), (1, 2), False), ((3, 4, 5, 6), (0, 2), True)])
def test_reduce_sum(shape, dims, keep):
    # tests/ut/test_reduce.py:22-107 (eps 1e-4)
    a = np.random.default_rng(3).normal(0, 1, shape).astype(np.float32)
    o = OracleKernel()
    got = o.store(o.sum(o.load(a), dims, keep))
    assert close(got, np.sum(a, axis=dims, keepdims=keep), 1e-4)
    assert o.sum(o.load(a.astype(np.float16)), dims, keep) is None   # only fp32 sums exist (src/dvm.cc:1538-1540)


def test_integer_pow_and_scalar_forms():
    # tests/ut/test_elemwise.py:233-245, 430-440
    a = np.random.default_rng(4).uniform(0.5, 2, [257]).astype(np.float32)
    o = OracleKernel()
    x = o.load(a)
    assert close(o.store(o.pow(x, 3)), a * a * a, 1e-5)
    assert close(o.store(o.sub(2.0, x)), 2.0 - a, 1e-5)
    assert close(o.store(o.div(1.0, x)), 1.0 / a, 1e-5)
    assert close(o.store(o.pow(2.0, x)), np.power(2.0, a), 1e-5)


def test_examples_batchnorm_attention_matmul():
    # examples/02_batchnorm.py:19-60 (eps 1e-3), 03_attention.py:20-63 (1e-2), 04_matmul_post_fusion.py:50-58 (1e-2)
    rng = np.random.default_rng(5)
    x = rng.normal(size=(4, 8, 6, 6)).astype(np.float16)
    gamma = rng.normal(1, 0.1, (1, 8, 1, 1)).astype(np.float32)
    beta = rng.normal(0, 0.1, (1, 8, 1, 1)).astype(np.float32)
    o = OracleKernel()
    y, mean, var = (o.store(v) for v in W.batchnorm_train(o, o.load(x), o.load(gamma), o.load(beta), 4 * 36))
    xf = x.astype(np.float32)
    m, v = xf.mean(axis=(0, 2, 3), keepdims=True), xf.var(axis=(0, 2, 3), keepdims=True)
    assert close(mean, m, 1e-4) and close(var, v, 1e-4)
    assert close(y, (xf - m) / np.sqrt(v + 1e-5) * gamma + beta, 2e-3)
    q, k, vv = (rng.normal(size=(4, 8)).astype(np.float16) for _ in range(3))
    got = o.store(W.attention(o, o.load(q), o.load(k), o.load(vv), 0.35, F16)).astype(np.float32)
    s = q.astype(np.float32) @ k.astype(np.float32).T * 0.35
    p = np.exp(s - s.max(-1, keepdims=True))
    assert close(got, (p / p.sum(-1, keepdims=True)) @ vv.astype(np.float32), 1e-2)
    a, b = rng.normal(0, 0.3, (16, 32)).astype(np.float16), rng.normal(0, 0.3, (32, 24)).astype(np.float16)
    c = o.cast(o.matmul(o.load(a), o.load(b), False, False), F32)
    got = o.store(o.div(c, o.add(o.exp(o.mul(c, -1.0)), 1.0)))
    ref = a.astype(np.float32) @ b.astype(np.float32)
    assert close(got, ref / (1 + np.exp(-ref)), 1e-2)


def test_golden_fixtures_match_the_oracle():
    from tests.golden.make_golden import cases
    data = np.load(os.path.join(HERE, "golden", "oracle_golden.npz"))
    for name, outs in cases().items():
        for i, out in enumerate(outs):
            want = data["%s_%d" % (name, i)]
            got = out.view(np.uint16) if str(out.dtype) == "bfloat16" else out
            assert got.dtype == want.dtype and got.shape == want.shape, name
            assert np.array_equal(got, want, equal_nan=got.dtype.kind == "f"), name
