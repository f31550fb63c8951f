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
    # the variance of a 16-bit tensor needs no pass of its own: sum and sum of squares of the deviations from each
    # channel's first element are taken together, so the tensor is read twice instead of three times
    assert len(bodies) == 2
    assert bodies[0][0] == "lda.fp16+Sub.s+ReduceSum.p0+Sqr+ReduceSum.p1"
    assert bodies[1][0] == "lda.fp16+Sub.s+Mul.s+Mul.s+Add.s+st.fp16"
    # every body is one micro-op that runs all eight rounds of a chunk in one dispatch
    assert "rounds=8" in k.das()
    assert all(len(body) == 9 and " ".join(body).endswith("(ends the body, loops over the chunk's rounds)") for body in bodies)

    k = dvm.PyKernel("vector", "das", 0)
    T = 256
    h, r, gg, u = (k.load([T, 4096], dvm.bfloat16) for _ in range(4))
    w = k.load([4096], dvm.bfloat16)
    for o in W.rmsnorm_swiglu(k, h, r, w, gg, u, 4096):
        k.store(o)
    k.codegen()
    bodies = _micro_ops(k.das())
    # the residual RMSNorm + gated activation: three dispatches per 16 elements in all
    assert bodies[0][:2] == ["lda.bf16+ldb+Add.b+Sqr+ReduceSum.p0", "lda.bf16+SigmoidFast+ldb+Mul.b+ldb+Mul.b+st.bf16"]
    assert bodies[1][0] == "lda.bf16+ldb+Add.b+Mul.s+ldb+Mul.b+st.bf16"


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


def test_deviation_sums_keep_their_own_pass_on_request():
    # DVM_B200_EXACT_MATH=1 keeps a graph's reductions as written: mean, then the squared deviations from it, then the
    # result (three passes); a fp32 input is never rewritten either
    import subprocess, sys
    code = ("import sys, dvm_b200 as dvm\n"
            "from dvm_b200 import workloads as W\n"
            "dt = dvm.float16 if sys.argv[1] == 'f16' else dvm.float32\n"
            "k = dvm.PyKernel('vector', 'das', 0)\n"
            "x = k.load([8, 32, 14, 14], dt); g = k.load([1, 32, 1, 1], dvm.float32); b = k.load([1, 32, 1, 1], dvm.float32)\n"
            "[k.store(o) for o in W.batchnorm_train(k, x, g, b, 8 * 14 * 14)]\n"
            "k.codegen(); print(k.das())\n")

    def bodies(dtype, **extra):
        env = dict(os.environ, PYTHONPATH=ROOT, **extra)
        out = subprocess.run([sys.executable, "-c", code, dtype], env=env, capture_output=True, text=True, check=True).stdout
        return sum(1 for line in out.splitlines() if line.strip().startswith("body_") and line.strip().endswith(":"))

    assert bodies("f16") == 2
    assert bodies("f16", DVM_B200_EXACT_MATH="1") == 3
    assert bodies("f32") == 3


def _reloc_array(pairs):
    arr = (_capi.Reloc * len(pairs))()
    for i, (op, addr) in enumerate(pairs):
        arr[i].io = op._h
        arr[i].addr = addr
    return arr


def test_ring_slot_comes_back_after_an_unaligned_rebind(lib):
    # a tensor planned for bulk staging loses its ring slot while it is bound to an address that is not 16-byte aligned,
    # and gets the planned slot back (not a stale marker) when it is bound to an aligned address again
    k = dvm.PyKernel("vector", "das", 0)
    a = k.load([64, 4096], dvm.float32)
    b = k.load([64, 4096], dvm.float32)
    s = k.store(k.add(a, b))
    ws = ctypes_size_t()
    assert lib.dvm_pre_codegen(k._k, ws) == 0

    def listing(addr_a):
        rel = _reloc_array([(a, addr_a), (b, 0x20000000), (s, 0x30000000)])
        lib.dvm_launch_reloc(k._k, rel, len(rel), None, None)   # binds, then fails to launch without a device
        return k.das()

    aligned = listing(0x10000000)
    assert "t0: fp32 dense vec=1 ring=1" in aligned and "staged: body_0=0x3" in aligned
    unaligned = listing(0x10000004)
    assert "t0: fp32 dense vec=0 ring=0" in unaligned and "staged: body_0=0x2" in unaligned
    again = listing(0x10000000)
    assert again == aligned


def ctypes_size_t():
    import ctypes
    return ctypes.byref(ctypes.c_size_t(0))


def test_static_scratch_launch_reads_the_workspace_of_the_current_program(lib):
    # the capacity check must see the program compiled for the shapes of NOW, also when the last compile was triggered
    # by a listing after a shape update and not by dvm_pre_codegen / dvm_codegen
    k = dvm.PyKernel("split:dyn", "das", 0)
    sa, sb = dvm.IntArrayRef([128, 64]), dvm.IntArrayRef([128, 64])
    a, b = k.load(sa, dvm.bfloat16), k.load(sb, dvm.bfloat16)
    prod = k.cast(k.matmul(a, b, False, True), dvm.float32)
    s1, s2 = k.store(k.sum(prod, (1,), True)), k.store(k.mul(prod, 2.0))
    ws = ctypes_size_t()
    assert lib.dvm_pre_codegen(k._k, ws) == 0
    small = ws._obj.value
    assert 0 < small <= lib.dvm_static_scratch_capacity()
    sa.update([4096, 64])
    sb.update([2048, 64])           # fp32 product of 4096 x 2048: 32 MiB of workspace
    assert lib.dvm_normalize(k._k) == 0
    k.das()                         # compiles for the new shapes
    rel = _reloc_array([(a, 0x10000000), (b, 0x20000000), (s1, 0x30000000), (s2, 0x40000000)])
    rc = lib.dvm_launch_static_scratch(k._k, rel, len(rel), None)
    assert rc == -2 and "static scratch" in _capi.last_error()
    # and a kernel that was never compiled for its current shapes is refused outright
    sa.update([256, 64])
    sb.update([256, 64])
    assert lib.dvm_normalize(k._k) == 0
    assert lib.dvm_launch_static_scratch(k._k, rel, len(rel), None) == -5


def test_sequence_kernel_cuts_a_stage_at_every_seq_add():
    # Kernel::SequenceAdd (include/dvm.h:559): ops after the call form the next stage, launched after the previous one
    k = dvm.PyKernel("seq", "das", 0)
    k.seq_add(k.K_VEC)
    a = k.load([1024, 128], dvm.float32)
    c = k.mul(a, k.add(a, 0.2))
    k.seq_add(k.K_VEC)
    k.store(k.mul(c, 0.7))
    k.codegen()
    das = k.das()
    assert das.count("vmain") == 2
    assert "workspace_bytes=%d" % (1024 * 128 * 4) in k.inspect()
    with pytest.raises(RuntimeError):
        k.seq_add(k.K_SEQ)          # "invalid sequence add kernel type"
    with pytest.raises(RuntimeError):
        dvm.PyKernel("vector", "das", 0).seq_add(0)


def test_parallel_kernel_keeps_its_sub_kernels_apart():
    # Kernel::ParallelAdd (include/dvm.h:552): independent sub-kernels, one set of launches each
    k = dvm.PyKernel("parallel", "das", 0)
    for n, f in ((256, 0.3), (8192, 0.5), (1024, 0.7)):
        k.parallel_add(k.K_VEC)
        k.store(k.mul(k.load([n], dvm.float32), f))
    k.codegen()
    assert k.das().count("vmain") == 3
    with pytest.raises(RuntimeError):
        dvm.PyKernel("vector", "das", 0).parallel_add(0)
    # a sub-kernel may hold a MatMul (kCube / kMix); a stacked kernel type as sub-kernel is refused
    k.parallel_add(k.K_MIX)
    a, b = k.load([128, 64], dvm.float16), k.load([64, 256], dvm.float16)
    k.store(k.matmul(a, b, False, False))
    k.codegen()
    assert k.das().count("vmain") == 3 and k.das().count("mmain") == 1
    with pytest.raises(RuntimeError):
        k.parallel_add(3)


def test_spec_next_and_inplace_mark_are_checked():
    k = dvm.PyKernel("vector:spec", "das", 0)
    a = k.load([10, 6000], dvm.float32)
    r = k.sum(k.add(a, 0.02), (0,), True)
    k.spec_next()                                   # a stage hint: accepted, the result does not depend on it
    s = k.store(k.mul(r, a))
    k.set_store_inplace(s)
    k.codegen()
    assert k.das().count("vmain") == 1
    with pytest.raises(RuntimeError):
        dvm.PyKernel("vector", "das", 0).spec_next()   # only speculative vector kernels have stages to advance
    with pytest.raises(RuntimeError):
        k.set_store_inplace(a)                      # not a store


def test_views_carry_their_strides_into_the_tensor_table():
    # Kernel::Load(addr, shape, stride, type) / Store(addr, input, stride): include/dvm.h:294, 339
    k = dvm.PyKernel("vector", "das", 0)
    x = k.view_load([64, 32, 56, 56], [256 * 3136, 3136, 56, 1], dvm.float16)     # 32 channels of an NCHW [64,256,56,56]
    k.view_store(k.mul(x, 2.0), [256 * 3136, 3136, 56, 1])
    k.codegen()
    das = k.das()
    assert das.count("estride=[0,802816,3136,1]") + das.count("estride=[0,0,802816,1]") >= 2, das[:600]
    # strides that describe a contiguous tensor are an ordinary load
    k = dvm.PyKernel("vector", "das", 0)
    k.store(k.add(k.view_load([8, 16], [16, 1], dvm.float32), 1.0))
    k.codegen()
    assert "mode=flat" in k.das() and "fp32 dense" in k.das()
    with pytest.raises(RuntimeError):
        k = dvm.PyKernel("vector", "das", 0)
        k.store(k.view_load([8, 16], [16], dvm.float32))      # one stride per dim
        k.codegen()


def test_view_ops_infer_shapes_and_plan_without_a_copy():
    # Kernel::Permute / Slice / Split are views of a tensor in memory (include/dvm.h:428-453, 470-479)
    k = dvm.PyKernel("vector", "das", 0)
    x = k.load([6, 40, 96], dvm.float32)
    p = k.permute(x, [2, 0, 1])
    s = k.slice(x, [1, 8, 16], [4, 20, 64])
    d = k.slice_dim(x, 1, -10, 40)
    chunks = k.split(x, 2, 40, 3)
    for v in [p, s, d] + chunks:
        k.store(k.add(v, 1.0))
    k.codegen()
    assert p.shape() == (96, 6, 40) and s.shape() == (4, 20, 64) and d.shape() == (6, 10, 96)
    assert [c.shape() for c in chunks] == [(6, 40, 40), (6, 40, 40), (6, 40, 16)]
    assert "workspace_bytes=0" in k.inspect()          # no copies: every view reads the Load's own memory
    with pytest.raises(RuntimeError):
        bad = dvm.PyKernel("vector", "das", 0)
        bad.store(bad.slice(bad.load([4, 4], dvm.float32), [2, 2], [4, 4]))
        bad.codegen()


def test_concat_is_planned_as_slabs_of_one_workspace_tensor():
    # Kernel::Concat: every input is written to its slab by a launch of its own (a strided store), the ops behind the result
    # read the whole tensor; inputs must agree outside the concatenated dimension
    k = dvm.PyKernel("vector", "das", 0)
    a, b, c = k.load([8, 100], dvm.float32), k.load([8, 28], dvm.float32), k.load([8, 1], dvm.float32)
    cat = k.concat([k.add(a, 1.0), b, c], 1)
    k.store(k.mul(cat, 2.0))
    k.codegen()
    assert list(cat.shape()) == [8, 129]
    das = k.das()
    # the first input's add and its slab store are one launch; the workspace holds the concatenated tensor and nothing else
    assert das.count("vmain.") == 4 and "workspace_bytes=%d" % ((8 * 129 * 4 + 255) // 256 * 256) in k.inspect()
    bad = dvm.PyKernel("vector", "das", 0)
    bad.store(bad.concat([bad.load([8, 100], dvm.float32), bad.load([7, 100], dvm.float32)], 1))
    with pytest.raises(Exception, match="concat inputs differ"):
        bad.codegen()


def test_slice_loads_are_strided_loads_with_an_offset():
    # Kernel::SliceLoad / StridedSliceLoad: the window's shape, the tensor's strides (times the steps) and the start as an
    # address offset; a window outside the tensor is refused
    k = dvm.PyKernel("vector", "das", 0)
    x = k.slice_load([32, 64], [3, 8], [16, 32], dvm.float32)
    y = k.stridedslice_load([32, 64], [-4, 0], [100, 64], [1, 2], dvm.float32)
    k.store(k.mul(x, 2.0))
    k.store(k.mul(y, 2.0))
    k.codegen()
    assert list(x.shape()) == [16, 32] and list(y.shape()) == [4, 32]
    bad = dvm.PyKernel("vector", "das", 0)
    bad.store(bad.mul(bad.slice_load([32, 64], [3, 40], [16, 32], dvm.float32), 2.0))
    with pytest.raises(Exception, match="slice outside its tensor"):
        bad.codegen()


def test_a_cloned_kernel_is_the_same_program_with_its_own_shapes():
    # Kernel::Clone (include/dvm.h:255-259): the copy compiles to the same program; its shapes and scalars are its own
    base = dvm.PyKernel("vector:dyn", "das", 0)
    x = base.load([-1, -1], dvm.float32)
    dims = dvm.IntArrayRef([0])
    s = base.store(base.sum(base.add(x, 0.01), dims, True))
    base.input(x, np.zeros((10, 512), np.float32))
    base.codegen()
    copy = dvm.PyKernel("", "das", 0)
    x2, s2, dims2 = copy.clone(base, [x, s, dims])
    copy.input(x2, np.zeros((10, 512), np.float32))
    copy.codegen()
    strip = lambda das: re.sub(r"@0x[0-9a-f]+|0x[0-9a-f]{4,}", "@", das)
    assert strip(copy.das()) == strip(base.das())
    assert list(s2.shape()) == [1, 512]
    dims2.update([1])                               # the copy's reduce dims are its own
    copy.input(x2, np.zeros((64, 800), np.float32))
    copy.codegen()
    assert list(s2.shape()) == [64, 1] and list(s.shape()) == [1, 512]
