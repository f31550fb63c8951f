"""Generates tests/golden/oracle_golden.npz: outputs of the CPU oracle on small seeded instances of the five benchmark
graphs and of the bit-exact op classes.  Run `python -m tests.golden.make_golden` from the repository root.

The reference holds no golden vectors for this path and cannot execute without a GPU, so these vectors come from the
oracle (itself pinned to the reference's test formulas in tests/test_oracle_pins.py).  They freeze the oracle and give
the device tests a fixed target that does not depend on the oracle's code at test time.
"""
import os

import numpy as np

from dvm_b200 import workloads as W

BF16, F16, F32, I32 = 2, 1, 3, 4   # dvm::DataType codes


def inputs():
    """name -> (list of input arrays, list of dtype codes or None)."""
    r = np.random.default_rng(2026)
    d = {}
    d["c1"] = ([r.uniform(-1, 1, (37, 515)).astype(np.float32) for _ in range(2)], [None, None])
    d["c2"] = ([r.standard_normal((4, 8, 7, 7)).astype(np.float16), r.normal(1, 0.1, (1, 8, 1, 1)).astype(np.float32),
                r.normal(0, 0.1, (1, 8, 1, 1)).astype(np.float32)], [None, None, None])
    d["c3"] = ([r.standard_normal((9, 512)).astype(np.float32), r.standard_normal((9, 512)).astype(np.float32),
                r.normal(1, 0.02, (512,)).astype(np.float32), r.standard_normal((9, 512)).astype(np.float32),
                r.standard_normal((9, 512)).astype(np.float32)], [BF16] * 5)
    d["c4"] = ([r.standard_normal((2, 3, 130, 64)).astype(np.float32) for _ in range(3)], [BF16] * 3)
    d["c5"] = ([r.normal(0, 0.05, (136, 72)).astype(np.float32), r.normal(0, 0.05, (72, 264)).astype(np.float32),
                r.normal(0, 0.05, (264,)).astype(np.float32)], [BF16] * 3)
    d["exact"] = ([r.normal(0, 40, (300,)).astype(np.float32), r.normal(0, 40, (300,)).astype(np.float32),
                   r.integers(-1000, 1000, (300,)).astype(np.int32)], [None, None, None])
    return d


def build(name, k, ops):
    if name == "c1":
        return [W.fused_elementwise(k, *ops)]
    if name == "c2":
        return list(W.batchnorm_train(k, *ops, 4 * 49))
    if name == "c3":
        return list(W.rmsnorm_swiglu(k, *ops, 512))
    if name == "c4":
        return [W.attention(k, *ops, 0.125)]
    if name == "c5":
        return [W.matmul_bias_gelu(k, *ops)]
    a, b, i = ops   # the bit-exact class: compare, select, casts, integer arithmetic
    return [k.greater(a, b), k.select(k.less_equal(a, b), a, b), k.cast(a, I32), k.cast(k.cast(a, F16), F32),
            k.add(k.mul(i, i), 7), k.cast(i, F32), k.maximum(a, b), k.cast(a, BF16)]


def cases():
    from oracle.dvm_oracle import OracleKernel
    out = {}
    for name, (arrays, dts) in inputs().items():
        o = OracleKernel()
        out[name] = [o.store(v) for v in build(name, o, [o.load(a, d) for a, d in zip(arrays, dts)])]
    return out


def main():
    flat = {}
    for name, outs in cases().items():
        for i, a in enumerate(outs):
            flat["%s_%d" % (name, i)] = a.view(np.uint16) if str(a.dtype) == "bfloat16" else a
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_golden.npz")
    np.savez_compressed(path, **flat)
    print(path, os.path.getsize(path), "bytes,", len(flat), "arrays")


if __name__ == "__main__":
    main()
