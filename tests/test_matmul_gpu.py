"""Device parity of the MatMul stage (tcgen05 kernel, SIMT kernel, fused post-ops) against the NumPy oracle,
through the C ABI.  Shapes follow the reference's MatMul tests (tests/ut/test_matmul.py: plain, transposed,
bias row broadcast, post-fusion, unaligned, batched with broadcast)."""
import numpy as np
import pytest

from dvm_b200 import workloads as W
from tests.util import BF16, TOL_HALF, assert_close, run_both

pytestmark = pytest.mark.gpu

BF, F16 = 2, 1


def _mats(rng, m, n, k, ta=False, tb=False, batch_a=(), batch_b=(), scale=0.1):
    a = rng.normal(0, scale, batch_a + ((k, m) if ta else (m, k))).astype(np.float32)
    b = rng.normal(0, scale, batch_b + ((n, k) if tb else (k, n))).astype(np.float32)
    return a, b


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (100, 72, 40), (1, 8, 8),
                                   (130, 264, 72), (1024, 1024, 512), (2048, 4096, 256)])
@pytest.mark.parametrize("dt", [BF, F16])
def test_plain_matmul(m, n, k, dt):
    rng = np.random.default_rng(5)
    a, b = _mats(rng, m, n, k)
    dev, ref, t = run_both(lambda kk, x, y: kk.matmul(x, y, False, False), [a, b], ker_type="mix", dtypes=[dt, dt])
    assert "tcgen05" in t.das()
    assert_close(dev[0], ref[0], TOL_HALF, "matmul %dx%dx%d" % (m, n, k))


@pytest.mark.parametrize("ta,tb", [(False, True), (True, False), (True, True)])
def test_transposed_operands(ta, tb):
    rng = np.random.default_rng(6)
    a, b = _mats(rng, 192, 320, 136, ta, tb)
    dev, ref, t = run_both(lambda kk, x, y: kk.matmul(x, y, ta, tb), [a, b], ker_type="mix", dtypes=[BF, BF])
    assert "tcgen05" in t.das()
    assert_close(dev[0], ref[0], TOL_HALF, "matmul ta=%s tb=%s" % (ta, tb))


@pytest.mark.parametrize("m,n,k", [(33, 17, 29), (64, 30, 64), (5, 7, 3)])
def test_unaligned_shapes_run_on_the_simt_kernel(m, n, k):
    rng = np.random.default_rng(7)
    a, b = _mats(rng, m, n, k)
    dev, ref, t = run_both(lambda kk, x, y: kk.matmul(x, y, False, False), [a, b], ker_type="mix", dtypes=[BF, BF])
    assert "simt" in t.das()
    assert_close(dev[0], ref[0], TOL_HALF, "unaligned matmul")


def test_bias_and_gelu_post_fusion_is_one_launch():
    rng = np.random.default_rng(5)
    a = rng.normal(0, 0.02, (512, 1024)).astype(np.float32)
    b = rng.normal(0, 0.02, (1024, 768)).astype(np.float32)
    bias = rng.normal(0, 0.02, (768,)).astype(np.float32)
    dev, ref, t = run_both(W.matmul_bias_gelu, [a, b, bias], ker_type="mix", dtypes=[BF, BF, BF])
    das = t.das()
    assert das.count("mmain") == 1 and "vmain" not in das
    assert_close(dev[0], ref[0], TOL_HALF, "gelu(A B + bias)")
    # and against the plain formula
    c = a.astype(BF16).astype(np.float32) @ b.astype(BF16).astype(np.float32) + bias.astype(BF16).astype(np.float32)
    want = 0.5 * c * (1 + np.tanh(0.7978845608 * (c + 0.044715 * c ** 3)))
    assert_close(dev[0], want, 2e-2, "gelu vs numpy tanh form")


def test_post_fusion_with_full_and_column_operands_and_two_outputs():
    rng = np.random.default_rng(8)
    a, b = _mats(rng, 200, 136, 64)
    res = rng.normal(size=(200, 136)).astype(np.float32)
    col = rng.normal(size=(200, 1)).astype(np.float32)

    def build(k, x, y, r, c):
        p = k.cast(k.matmul(x, y, False, False), 3)
        q = k.add(k.mul(p, c), r)
        return k.cast(q, BF), k.maximum(q, 0.0)

    dev, ref, t = run_both(build, [a, b, res, col], ker_type="mix", dtypes=[BF, BF, None, None])
    assert t.das().count("mmain") == 1 and "vmain" not in t.das()
    assert_close(dev[0], ref[0], TOL_HALF, "residual epilogue bf16")
    assert_close(dev[1], ref[1], TOL_HALF, "relu output fp32")


def test_batched_with_broadcast_rhs():
    rng = np.random.default_rng(9)
    a, b = _mats(rng, 96, 80, 64, batch_a=(3, 2), batch_b=(2,))
    dev, ref, _ = run_both(lambda kk, x, y: kk.matmul(x, y, False, False), [a, b], ker_type="mix", dtypes=[BF, BF])
    assert dev[0].shape == (3, 2, 96, 80)
    assert_close(dev[0], ref[0], TOL_HALF, "batched matmul")


def test_matmul_feeding_a_reduction_is_split_into_stages():
    rng = np.random.default_rng(10)

    def build(k, x, y):
        p = k.cast(k.matmul(x, y, False, True), 3)
        return k.sum(p, (1,), True)

    a2, b2 = _mats(rng, 64, 128, 64, tb=True)
    dev, ref, t = run_both(build, [a2, b2], ker_type="split", dtypes=[BF, BF])
    assert t.das().count("mmain") == 1 and t.das().count("vmain") == 1
    assert_close(dev[0], ref[0], TOL_HALF, "row sums of a product")


def test_config5_rows_at_full_size():
    """The full MatMul + bias + GeLU workload [16384 x 8192 x 8192]; a sample of rows is checked exactly against
    the oracle, the rest through finiteness and a column checksum of the sampled rows."""
    rng = np.random.default_rng(5)
    m, n, k = 16384, 8192, 8192
    a = rng.normal(0, 0.02, (m, k)).astype(np.float32).astype(BF16)
    b = rng.normal(0, 0.02, (k, n)).astype(np.float32).astype(BF16)
    bias = rng.normal(0, 0.02, (n,)).astype(np.float32).astype(BF16)
    from dvm_b200.tester import Tester
    from oracle.dvm_oracle import OracleKernel
    t = Tester("mix")
    s = t.store(W.matmul_bias_gelu(t, t.load(a), t.load(b), t.load(bias)))
    t.run()
    got = t.output(s).astype(np.float32)
    assert np.isfinite(got).all()
    rows = np.concatenate([np.arange(0, 8), rng.integers(0, m, 48), np.arange(m - 8, m)])
    o = OracleKernel()
    want = o.store(W.matmul_bias_gelu(o, o.load(a[rows]), o.load(b), o.load(bias))).astype(np.float32)
    assert_close(got[rows], want, TOL_HALF, "sampled rows of the full-size product")
