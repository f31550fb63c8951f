"""The peephole pass of the vector compiler must not change a single bit: every fused micro-op performs its parts'
operations in their order, each rounded on its own.  The same graphs run in two fresh processes, with the pass and
without it (it is read once per process), and the outputs are compared bit for bit."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys
import numpy as np
import ml_dtypes
from dvm_b200 import workloads as W
from dvm_b200.tester import Tester

BF16 = np.dtype(ml_dtypes.bfloat16)
out = {}
fused_seen = 0


def run(name, build, arrays, dtypes=None):
    global fused_seen
    t = Tester("vector")
    dtypes = dtypes or [None] * len(arrays)
    vals = build(t, *[t.load(a, d) for a, d in zip(arrays, dtypes)])
    vals = vals if isinstance(vals, (tuple, list)) else (vals,)
    stores = [t.store(v) for v in vals]
    t.run()
    fused_seen += t.das().count("+")
    for i, s in enumerate(stores):
        a = np.asarray(t.output(s))
        out["%s_%d" % (name, i)] = a.view(np.uint16) if a.dtype == BF16 else a


rng = np.random.default_rng(11)
# batch-norm statistics and normalisation on strided fp16 planes (load + reduce, load - scalar, square + reduce,
# scalar-register triple, rounding folded into the store)
x = rng.standard_normal((8, 24, 28, 28), dtype=np.float32).astype(np.float16)
g = rng.normal(1, 0.1, (1, 24, 1, 1)).astype(np.float32)
b = rng.normal(0, 0.1, (1, 24, 1, 1)).astype(np.float32)
run("bn", lambda k, a, c, d: W.batchnorm_train(k, a, c, d, 8 * 28 * 28), [x, g, b])
# the same on planes of 56 x 56 (chunks of several rounds, every body one looping micro-op), with a last chunk that is
# not full (19 planes, 8 per chunk)
x = rng.standard_normal((19, 6, 56, 56), dtype=np.float32).astype(np.float16)
run("bn_rounds", lambda k, a, c, d: W.batchnorm_train(k, a, c, d, 19 * 56 * 56), [x, g[:, :6], b[:, :6]])
# residual + RMSNorm + SwiGLU in bf16 (two ring operands + add, ring operand + mul, fast sigmoid), rows with a ragged tail
for rows, hidden in ((37, 4096), (5, 1000)):
    h, r, gg, u = (rng.standard_normal((rows, hidden), dtype=np.float32).astype(BF16) for _ in range(4))
    w = rng.normal(1, 0.02, (hidden,)).astype(np.float32).astype(BF16)
    run("rms%d" % hidden, lambda k, a, c, d, e, f, n=hidden: W.rmsnorm_swiglu(k, a, c, d, e, f, n), [h, r, w, gg, u])
# the same graph on fp16 and fp32 storage (the fused sum-of-squares, scaled-sum and gated-activation forms of each type)


def rms_any(k, a, c, d, e, f, n, dt):
    s = k.add(k.cast(a, 3), k.cast(c, 3))
    inv = k.div(1.0, k.sqrt(k.add(k.mul(k.sum(k.mul(s, s), (1,), True), 1.0 / n), 1e-6)))
    o1 = k.cast(k.mul(k.mul(s, inv), k.cast(d, 3)), dt)
    ef = k.cast(e, 3)
    o2 = k.cast(k.mul(k.mul(ef, k.div(1.0, k.add(k.exp(k.mul(ef, -1.0)), 1.0))), k.cast(f, 3)), dt)
    return o1, o2


for dt, code, tag in ((np.float16, 1, "f16"), (np.float32, 3, "f32")):
    h, r, gg, u = (rng.standard_normal((21, 2048), dtype=np.float32).astype(dt) for _ in range(4))
    w = rng.normal(1, 0.02, (2048,)).astype(dt)
    run("rms_" + tag, lambda k, a, c, d, e, f, c_=code: rms_any(k, a, c, d, e, f, 2048, c_), [h, r, w, gg, u])
# reduce-free chains in the three storage types
for dt, tag in ((np.float32, "f32"), (np.float16, "f16")):
    p = rng.uniform(-2, 2, (333, 2048)).astype(dt)
    q = rng.uniform(0.5, 2, (333, 2048)).astype(dt)
    run("chain_" + tag, lambda k, a, c: (k.add(k.mul(k.sub(a, c), c), a), k.mul(k.add(a, c), k.sub(a, c))), [p, q])
run("exp_f32", W.fused_elementwise, [rng.uniform(-1, 1, (1024, 4096)).astype(np.float32),
                                      rng.uniform(-1, 1, (1024, 4096)).astype(np.float32)])
# MatMul + bias + tanh-GeLU: the launcher recognises the post-fusion program and the kernel computes it in registers
# instead of interpreting it; rows / columns that do not fill a tile take the interpreter in both runs
for dt, code, tag in ((BF16, 2, "bf16"), (np.float16, 1, "f16")):
    for (m, n, kk) in ((256, 512, 128), (200, 264, 96)):
        a_ = rng.normal(0, 0.5, (m, kk)).astype(np.float32).astype(dt)
        b_ = rng.normal(0, 0.5, (kk, n)).astype(np.float32).astype(dt)
        bias_ = rng.normal(0, 0.5, (n,)).astype(np.float32).astype(dt)
        t = Tester("mix")
        la, lb, lbias = t.load(a_), t.load(b_), t.load(bias_)
        c = t.matmul(la, lb, False, False, lbias)
        st = t.store(t.cast(W.gelu_tanh(t, t.cast(c, 3)), code))
        t.run()
        o = np.asarray(t.output(st))
        out["mm_gelu_%s_%d" % (tag, m)] = o.view(np.uint16)
np.savez(sys.argv[1], fused_seen=np.int64(fused_seen), **out)
"""


def _run_child(path, extra_env):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    env.pop("DVM_B200_NO_FUSE", None)
    env.pop("DVM_B200_NO_TAIL", None)
    env.update(extra_env)
    subprocess.run([sys.executable, "-c", CHILD, path], env=env, check=True, cwd=ROOT, timeout=600)
    return dict(np.load(path))


def test_fused_program_equals_unfused_bit_for_bit(tmp_path):
    fused = _run_child(str(tmp_path / "fused.npz"), {})
    plain = _run_child(str(tmp_path / "plain.npz"), {"DVM_B200_NO_FUSE": "1", "DVM_B200_NO_TAIL": "1"})
    assert int(fused.pop("fused_seen")) > 0 and int(plain.pop("fused_seen")) == 0
    assert sorted(fused) == sorted(plain) and len(fused) >= 10
    for name in sorted(fused):
        a, b = fused[name], plain[name]
        assert a.dtype == b.dtype and a.shape == b.shape, name
        assert a.tobytes() == b.tobytes(), "%s: fused and unfused programs differ in %d elements" % (
            name, int((a.view(np.uint8) != b.view(np.uint8)).sum()))
