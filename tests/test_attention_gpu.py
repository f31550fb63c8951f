"""Device parity of the attention pattern MatMul -> scale -> softmax -> MatMul (examples/03_attention.py:31-52 of
the reference, with batch dims) against the NumPy oracle, through the C ABI: the fused tcgen05 kernel where the
head dimension allows it, the MatMul / vector / MatMul stage sequence otherwise."""
import numpy as np
import pytest

from dvm_b200 import workloads as W
from tests.util import BF16, TOL_HALF, assert_close, run_both

pytestmark = pytest.mark.gpu

BF, F16 = 2, 1


def _qkv(rng, batch, sq, skv, d):
    q = rng.standard_normal(batch + (sq, d)).astype(np.float32)
    k = rng.standard_normal(batch + (skv, d)).astype(np.float32)
    v = rng.standard_normal(batch + (skv, d)).astype(np.float32)
    return q, k, v


@pytest.mark.parametrize("batch,sq,skv,d,dt", [
    ((2, 2), 256, 256, 128, BF),
    ((1, 3), 128, 384, 128, BF),
    ((4,), 200, 333, 64, F16),
    ((), 512, 128, 64, BF),
    ((2, 1), 1, 77, 128, BF),
    ((1, 2), 700, 1000, 128, F16),
])
def test_fused_attention(batch, sq, skv, d, dt):
    rng = np.random.default_rng(4)
    q, k, v = _qkv(rng, batch, sq, skv, d)
    scale = 1.0 / np.sqrt(d)
    dev, ref, t = run_both(lambda kk, a, b, c: W.attention(kk, a, b, c, scale, dt), [q, k, v], ker_type="split",
                           dtypes=[dt, dt, dt])
    das = t.das()
    assert das.count("amain") == 1 and "vmain" not in das and "mmain" not in das
    assert_close(dev[0], ref[0], TOL_HALF, "attention %s %dx%dx%d" % (batch, sq, skv, d))
    # and against a plain fp32 softmax of the same rounded inputs
    def r(a):
        return a.astype(BF16 if dt == BF else np.float16).astype(np.float32)
    s = np.einsum("...qd,...kd->...qk", r(q), r(k)) * scale
    p = np.exp(s - s.max(-1, keepdims=True))
    want = np.einsum("...qk,...kd->...qd", p / p.sum(-1, keepdims=True), r(v))
    assert_close(dev[0], want, 2e-2, "attention vs plain softmax")


def test_attention_with_large_scores_rescales_the_accumulator():
    # keys grow along the sequence, so the running maximum rises by far more than the lazy-rescale threshold
    rng = np.random.default_rng(41)
    q, k, v = _qkv(rng, (2,), 256, 640, 128)
    k *= np.linspace(0.2, 6.0, 640, dtype=np.float32)[None, :, None]
    dev, ref, _ = run_both(lambda kk, a, b, c: W.attention(kk, a, b, c, 0.125), [q, k, v], ker_type="split", dtypes=[BF] * 3)
    assert_close(dev[0], ref[0], TOL_HALF, "attention with a rising maximum")


def test_unsupported_head_dim_runs_as_three_stages():
    rng = np.random.default_rng(42)
    q, k, v = _qkv(rng, (2,), 96, 160, 32)
    dev, ref, t = run_both(lambda kk, a, b, c: W.attention(kk, a, b, c, 0.2), [q, k, v], ker_type="split", dtypes=[BF] * 3)
    das = t.das()
    assert "amain" not in das and das.count("mmain") == 2 and das.count("vmain") == 1
    assert_close(dev[0], ref[0], TOL_HALF, "unfused attention")


def test_config4_heads_at_full_size():
    """Q, K, V bf16 [8, 32, 2048, 128]: the whole workload runs once; three (batch, head) slices are checked against
    the oracle and every output row against the convexity of softmax (each output lies inside the range of V)."""
    rng = np.random.default_rng(4)
    shape = (8, 32, 2048, 128)
    q, k, v = (rng.standard_normal(shape, dtype=np.float32).astype(BF16) for _ in range(3))
    scale = 1.0 / np.sqrt(128.0)
    from dvm_b200.tester import Tester
    from oracle.dvm_oracle import OracleKernel
    t = Tester("split")
    s = t.store(W.attention(t, t.load(q), t.load(k), t.load(v), scale))
    t.run()
    assert t.das().count("amain") == 1
    got = t.output(s).astype(np.float32)
    assert np.isfinite(got).all()
    vf = v.astype(np.float32)
    assert (got <= vf.max(axis=2, keepdims=True) + 1e-2).all() and (got >= vf.min(axis=2, keepdims=True) - 1e-2).all()
    for b, h in [(0, 0), (3, 17), (7, 31)]:
        o = OracleKernel()
        want = o.store(W.attention(o, o.load(q[b, h]), o.load(k[b, h]), o.load(v[b, h]), scale)).astype(np.float32)
        assert_close(got[b, h], want, TOL_HALF, "head (%d, %d) of the full-size workload" % (b, h))
