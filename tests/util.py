"""Helpers shared by the parity tests: run one graph definition on the device (through the C ABI) and on
the NumPy oracle, and compare under the tolerance classes of the benchmark contract."""
import numpy as np

from oracle.dvm_oracle import OracleKernel

try:
    import ml_dtypes
    BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    BF16 = None

# tolerance classes: bit-exact for integer/compare/select/cast, 1e-5 relative for fp32 elementwise,
# 1e-2 for fp16/bf16 and for reductions, attention and matmul
TOL_EXACT = 0.0
TOL_FP32 = 1e-5
TOL_HALF = 1e-2
TOL_REDUCE = 1e-2


def as_f32(a):
    a = np.asarray(a)
    if BF16 is not None and a.dtype == BF16:
        return a.astype(np.float32)
    if a.dtype == np.bool_:
        return a.astype(np.float32)
    return a.astype(np.float32) if a.dtype.kind == "f" else a


def assert_close(got, want, tol, what=""):
    got, want = as_f32(got), as_f32(want)
    assert got.shape == want.shape, "%s: shape %s vs %s" % (what, got.shape, want.shape)
    if tol == 0:
        same = (got == want) | (np.isnan(got.astype(np.float64)) & np.isnan(want.astype(np.float64)))
        assert same.all(), "%s: %d of %d elements differ (bit-exact class)" % (what, (~same).sum(), same.size)
    else:
        ok = np.isclose(got, want, rtol=tol, atol=tol, equal_nan=True)
        if not ok.all():
            i = tuple(np.argwhere(~ok)[0])
            raise AssertionError("%s: %d of %d outside tol %g; first at %s got %r want %r" %
                                 (what, (~ok).sum(), ok.size, tol, i, got[i], want[i]))


def run_both(build, arrays, ker_type="vector", dtypes=None):
    """build(k, *loaded) -> value or tuple of values.  Returns (device outputs, oracle outputs)."""
    from dvm_b200.tester import Tester
    dtypes = dtypes or [None] * len(arrays)
    t = Tester(ker_type)
    vals = build(t, *[t.load(a, d) for a, d in zip(arrays, dtypes)])
    vals = vals if isinstance(vals, (tuple, list)) else (vals,)
    stores = [t.store(v) for v in vals]
    t.run()
    dev = [t.output(s) for s in stores]
    o = OracleKernel()
    ovals = build(o, *[o.load(a, d) for a, d in zip(arrays, dtypes)])
    ovals = ovals if isinstance(ovals, (tuple, list)) else (ovals,)
    ref = [o.store(v) for v in ovals]
    return dev, ref, t
