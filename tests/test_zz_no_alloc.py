"""dvm_launch_static_scratch(): the launch for callers that may not allocate device memory at launch time (a
framework's allocator hook, a no-allocation region of a memory pool, a latency-critical serving path).  The
kernel's workspace then comes from a fixed array inside the library instead of a caller-provided buffer.

The graph below is split into two launches (MatMul, then a row reduction) that hand the product over through the
workspace, so the entry point really exercises scratch memory.  Its result must equal the regular
dvm_codegen()/dvm_launch() path on two calls in a row, and a kernel whose workspace is larger than the array
must be refused.  Collected last on purpose: a failure here cannot hide the other tests.
"""
import ctypes

import numpy as np
import pytest

from dvm_b200 import _capi
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _build(m, n, k):
    from dvm_b200.tester import Tester
    rng = np.random.default_rng(77)
    a = rng.normal(0, 0.1, (m, k)).astype(np.float32)
    b = rng.normal(0, 0.1, (n, k)).astype(np.float32)
    t = Tester("split")
    la, lb = t.load(a, 2), t.load(b, 2)
    prod = t.cast(t.matmul(la, lb, False, True), 3)
    stores = [t.store(t.sum(prod, (1,), True)), t.store(t.mul(prod, 2.0))]
    return t, [la, lb], stores


def _relocs(t, ops):
    arr = (_capi.Reloc * len(ops))()
    for i, op in enumerate(ops):
        arr[i].io = op._h
        arr[i].addr = t.device_ptr(op)
    return arr


def test_static_scratch_launch_matches_the_regular_path_twice():
    lib = _capi.load()
    t, loads, stores = _build(192, 256, 64)
    t.run()                                   # regular path: workspace from the allocator callback
    assert t.das().count("main") >= 2         # two launches, so the workspace is in use
    want = [t.output(s).copy() for s in stores]
    relocs = _relocs(t, loads + stores)
    import torch
    for call in range(2):
        for s in stores:                      # wipe the outputs so that a launch that did nothing cannot pass
            host = t.output(s)
            assert lib.dvm_rt_memset(t.device_ptr(s), 0, host.nbytes, None) == 0
        assert lib.dvm_rt_sync(None) == 0, _capi.last_error()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.dvm_launch_static_scratch(t._k, relocs, len(relocs), None)
        assert rc == 0, _capi.last_error()
        assert lib.dvm_rt_sync(None) == 0, _capi.last_error()
        if call == 1:
            # the first call on a device may trigger one-time set-up inside the CUDA runtime (function attributes, the
            # symbol lookup); from the second call on the device's free memory must not move at all
            assert torch.cuda.mem_get_info()[0] == free_before, "the launch changed the device's free memory"
        for s, w in zip(stores, want):
            assert_close(t.output(s), w, 0.0, "static-scratch launch, call %d" % call)


def test_static_scratch_refuses_a_workspace_beyond_its_capacity():
    lib = _capi.load()
    cap = lib.dvm_static_scratch_capacity()
    assert cap == 16 << 20
    t, loads, stores = _build(4096, 2048, 64)   # fp32 product: 32 MiB of workspace
    t.codegen()
    relocs = _relocs(t, loads + stores)
    rc = lib.dvm_launch_static_scratch(t._k, relocs, len(relocs), None)
    assert rc != 0
    assert "static scratch" in _capi.last_error()
