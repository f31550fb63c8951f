"""Cross-check against the reference itself: the same graphs evaluated by mindspore-ai/dvm's own CUDA backend
(compiled from the reference tree into oracle/_ref/ by oracle/build_ref.py) and by this library on the same GPU and
the same seeded inputs.  The reference's GPU backend runs vector kernels only (src/system.cc:290-294), so MatMul and
attention are not covered here.  Skipped when the module was not built (no reference tree at build time)."""
import numpy as np
import pytest

from dvm_b200 import workloads as W
from oracle import ref_backend
from tests.util import TOL_EXACT, TOL_FP32, TOL_HALF, TOL_REDUCE, assert_close

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(ref_backend.module() is None, reason="oracle/_ref/_dvm_py was not built")]


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


def test_fused_elementwise_chain():
    rng = np.random.default_rng(0)
    x, y = (rng.uniform(-1, 1, (257, 1031)).astype(np.float32) for _ in range(2))
    dev, ref = both(W.fused_elementwise, [x, y])
    assert_close(dev[0], ref[0], TOL_FP32, "exp(x)*y+0.5 against the reference backend")


def test_exact_class_is_bit_identical():
    rng = np.random.default_rng(1)
    a, b = (rng.normal(0, 40, (3, 1000)).astype(np.float32) for _ in range(2))
    i = rng.integers(-1000, 1000, (3, 1000)).astype(np.int32)

    def build(k, a, b, i):
        return (k.greater(a, b), k.select(k.less_equal(a, b), a, b), k.cast(a, 4), k.cast(k.cast(a, 1), 3),
                k.add(k.mul(i, i), 7), k.cast(i, 3), k.maximum(a, b), k.floor(a), k.isfinite(k.log(a)))

    dev, ref = both(build, [a, b, i])
    for d, r, what in zip(dev, ref, ["greater", "select", "f32->i32", "f32->f16->f32", "int mul/add", "i32->f32", "maximum",
                                     "floor", "isfinite(log)"]):
        assert_close(d, r, TOL_EXACT, what + " against the reference backend")


def test_batchnorm_against_the_reference_backend():
    rng = np.random.default_rng(2)
    x = rng.normal(size=(8, 16, 14, 14)).astype(np.float16)
    gamma = rng.normal(1, 0.1, (1, 16, 1, 1)).astype(np.float32)
    beta = rng.normal(0, 0.1, (1, 16, 1, 1)).astype(np.float32)
    dev, ref = both(lambda k, a, g, b: W.batchnorm_train(k, a, g, b, 8 * 196), [x, gamma, beta], theirs="split")
    assert_close(dev[0], ref[0], TOL_HALF, "bn y")
    assert_close(dev[1], ref[1], TOL_REDUCE, "bn mean")
    assert_close(dev[2], ref[2], TOL_REDUCE, "bn var")


def test_rmsnorm_swiglu_against_the_reference_backend():
    rng = np.random.default_rng(3)
    h, r, g, u = (rng.standard_normal((33, 1024)).astype(np.float32) for _ in range(4))
    w = rng.normal(1, 0.02, (1024,)).astype(np.float32)
    from dvm_b200.tester import Tester
    from dvm_b200.frontend import PyKernel
    t = Tester("vector:spec,dyn")
    ours = [t.store(v) for v in W.rmsnorm_swiglu(t, *[t.load(a, 2) for a in (h, r, w, g, u)], 1024)]
    t.run()
    k = ref_backend.RefKernel("split")
    theirs = [k.store(v) for v in W.rmsnorm_swiglu(k, *[k.load(a, 2) for a in (h, r, w, g, u)], 1024)]
    k.run()
    for so, st, what in zip(ours, theirs, ["rmsnorm", "swiglu"]):
        got = PyKernel.convert_from_bf16(t.output(so))
        want = k.output(st, bf16=True)
        assert_close(np.asarray(got, dtype=np.float32), np.asarray(want, dtype=np.float32), TOL_HALF, what)
