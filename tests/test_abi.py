"""CPU checks of the boundary: the shared library loads and exports every symbol include/dvm_c.h declares,
and graph building / shape inference / code generation work without a device."""
import os
import re

import numpy as np
import pytest

import dvm_b200 as dvm
from dvm_b200 import _capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_symbols_exported(lib):
    text = open(os.path.join(ROOT, "include", "dvm_c.h")).read()
    declared = set(re.findall(r"DVM_C_API[^;]*?\b(dvm_[a-z0-9_]+)\s*\(", text))
    assert len(declared) >= 50
    for name in sorted(declared):
        assert hasattr(lib, name), "symbol %s declared in dvm_c.h is not exported" % name
    assert declared == set(_capi.SIGNATURES), declared ^ set(_capi.SIGNATURES)


def test_shape_inference_and_dtypes():
    k = dvm.PyKernel("vector", "das", 0)
    a = k.load([4, 1, 8], dvm.float16)
    b = k.load([5, 8], dvm.float16)
    c = k.add(a, b)
    d = k.greater(c, 0.5)
    e = k.sum(k.cast(c, dvm.float32), (0, 2), False)
    k.store(c), k.store(d), k.store(e)
    k._lib.dvm_normalize(k._k)
    assert c.shape() == (4, 5, 8) and c.dtype() == dvm.float16
    assert d.dtype() == dvm.bool_
    assert e.shape() == (5,)
    # a sum of anything but fp32 is refused with a null object, like the reference
    assert k.sum(c, (0,), False) is None


def test_errors_surface_as_runtime_error():
    k = dvm.PyKernel("vector", "das", 0)
    a = k.load([4, 3], dvm.float32)
    b = k.load([5, 3], dvm.float32)
    k.store(k.add(a, b))
    with pytest.raises(RuntimeError):
        k.codegen()
    with pytest.raises(RuntimeError):
        dvm.PyKernel("nonsense", "das", 0)


def test_compare_select_emits_no_cast():
    # compare -> select of one dtype must not materialise a cast (promotion casts are peeled again)
    k = dvm.PyKernel("vector", "das", 0)
    a = k.load([64], dvm.float32)
    b = k.load([64], dvm.float32)
    k.store(k.select(k.greater(a, b), a, b))
    k.codegen()
    text = k.das().lower()
    assert "cvt" not in text and "select" in text


def test_integer_pow_is_a_multiply_chain():
    k = dvm.PyKernel("vector", "das", 0)
    a = k.load([64], dvm.float32)
    k.store(k.pow(a, 5))
    k.codegen()
    assert k.das().count("Mul.fp32") == 3 and "Pow" not in k.das()


def test_fused_graph_is_one_launch_with_one_load_per_input():
    k = dvm.PyKernel("vector", "das", 0)
    x = k.load([8192, 8192], dvm.float32)
    y = k.load([8192, 8192], dvm.float32)
    k.store(k.add(k.mul(k.exp(x), y), 0.5))
    k.codegen()
    das = k.das()
    assert das.count("vmain") == 1 and das.count("load.") == 2 and das.count("store.") == 1
    assert "algorithmic_bytes=805306368" in k.inspect()


def test_dynamic_shape_recompile_is_stateless():
    # re-using one dynamic kernel over a shape sequence gives the same bytecode as a fresh kernel
    def build(shape):
        k = dvm.PyKernel("vector:dyn", "das", 0)
        ref = dvm.IntArrayRef(shape)
        a = k.load(ref, dvm.float32)
        k.store(k.mul(k.sum(k.mul(a, a), (1,), True), 0.5))
        return k, ref
    k, ref = build([3, 17])
    for shape in ([3, 17], [128, 4096], [1, 7], [1000, 333]):
        ref.update(shape)
        k.codegen()
        fresh, _ = build(shape)
        fresh.codegen()
        assert k.das() == fresh.das()


def _micro_ops(das):
    """The per-body micro-op listings of a disassembly, as lists of names."""
    return [line.split("micro-ops:")[1].split() for line in das.splitlines() if "micro-ops:" in line]


def test_peephole_fuses_frequent_neighbours():
    # the launch program of a full chunk: neighbours the peephole pass knows become one micro-op, and a body that ends
    # in a vector store or a reduce accumulation carries no END word
    from dvm_b200 import workloads as W
    k = dvm.PyKernel("vector", "das", 0)
    x = k.load([64, 256, 56, 56], dvm.float16)
    g = k.load([1, 256, 1, 1], dvm.float32)
    b = k.load([1, 256, 1, 1], dvm.float32)
    for o in W.batchnorm_train(k, x, g, b, 64 * 56 * 56):
        k.store(o)
    k.codegen()
    bodies = _micro_ops(k.das())
    assert len(bodies) == 3
    assert bodies[0][0] == "lda.fp16+ReduceSum.p0"
    assert bodies[1][0] == "lda.fp16+Sub.s+Sqr+ReduceSum.p1"
    assert bodies[2][:2] == ["lda.fp16+Sub.s+Mul.s+Mul.s+Add.s", "st.fp16"]
    assert all(body[-3:] == ["(ends", "the", "body)"] for body in bodies)

    k = dvm.PyKernel("vector", "das", 0)
    T = 256
    h, r, gg, u = (k.load([T, 4096], dvm.bfloat16) for _ in range(4))
    w = k.load([4096], dvm.bfloat16)
    for o in W.rmsnorm_swiglu(k, h, r, w, gg, u, 4096):
        k.store(o)
    k.codegen()
    bodies = _micro_ops(k.das())
    assert bodies[0][:4] == ["lda.bf16+ldb+Add.b", "Sqr+ReduceSum.p0", "lda.bf16+SigmoidFast", "ldb.bf16+Mul.b+ldb+Mul.b"]
    assert bodies[1][0] == "lda.bf16+ldb+Add.b"


def test_peephole_can_be_switched_off(monkeypatch):
    # the unfused program is what the fused one must equal bit for bit; the switch keeps it reachable for comparison
    import subprocess, sys
    code = ("import dvm_b200 as dvm\n"
            "k = dvm.PyKernel('vector', 'das', 0)\n"
            "a = k.load([64, 4096], dvm.float32); b = k.load([64, 4096], dvm.float32)\n"
            "k.store(k.add(a, b)); k.codegen(); print(k.das())\n")
    env = dict(os.environ, DVM_B200_NO_FUSE="1", DVM_B200_NO_TAIL="1", PYTHONPATH=ROOT)
    plain = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, check=True).stdout
    env = dict(os.environ, PYTHONPATH=ROOT)
    fused = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, check=True).stdout
    assert _micro_ops(plain)[0] == ["lda.fp32", "ldb.fp32", "Add.b", "st.fp32"]
    assert _micro_ops(fused)[0][:2] == ["lda.fp32+ldb+Add.b", "st.fp32"]
