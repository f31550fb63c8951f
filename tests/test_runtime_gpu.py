"""Runtime behaviour around a launch, on the device and through the C ABI: relocating launches that move a tensor
between aligned and unaligned addresses, and the report of a bounded device wait that ran out.

No counterpart in the reference's tests: its GPU interpreter waits without a limit and has no relocating launch from
Python; the relocation contract itself is include/dvm.h:201-206, 590-599.
"""
import ctypes

import numpy as np
import pytest

from dvm_b200 import _capi
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def test_relocating_launches_between_aligned_and_unaligned_addresses():
    """The same compiled kernel launched with an input at a 16-byte aligned address, then 4 bytes further (the producer
    warp may not bulk-copy from there, so the tensor leaves the ring), then aligned again (it returns to the slot the
    compiler planned)."""
    import torch
    from dvm_b200.tester import Tester
    lib = _capi.load()
    rng = np.random.default_rng(11)
    n = 64 * 4096
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    t = Tester("vector")
    a, b = t.load(x), t.load(y)
    s = t.store(t.add(t.mul(a, 1.5), b))
    t.run()
    want = x * np.float32(1.5) + y
    assert_close(t.output(s), want, 1e-6, "regular launch")

    buf = torch.empty(n + 8, dtype=torch.float32, device="cuda")
    out = torch.empty(n, dtype=torch.float32, device="cuda")
    hx = torch.from_numpy(x)
    for shift in (0, 1, 0, 1, 0):
        view = buf[shift:shift + n]
        view.copy_(hx)
        out.zero_()
        torch.cuda.synchronize()
        rel = (_capi.Reloc * 3)()
        rel[0].io, rel[0].addr = a._h, view.data_ptr()
        rel[1].io, rel[1].addr = b._h, t.device_ptr(b)
        rel[2].io, rel[2].addr = s._h, out.data_ptr()
        assert lib.dvm_launch_reloc(t._k, rel, 3, None, None) == 0, _capi.last_error()
        assert lib.dvm_rt_sync(None) == 0, _capi.last_error()
        das = t.das()
        assert ("t0: fp32 dense vec=1 ring=1" in das) == (shift == 0), das[:400]
        assert_close(out.cpu().numpy(), want, 1e-6, "relocated launch, input shifted by %d floats" % shift)


def test_an_expired_device_wait_is_reported_once_and_does_not_touch_later_launches():
    """A one-thread kernel waits on a barrier that nothing signals, through the interpreters' bounded wait with a 30 ms
    limit.  The wait gives up, the kernel ends normally, the host reads the record (status code 15) exactly once, and a
    regular kernel launched afterwards runs with full-length waits and correct results."""
    from dvm_b200.tester import Tester
    lib = _capi.load()
    assert lib.dvm_rt_sync(None) == 0, _capi.last_error()
    assert lib.dvm_rt_selftest_wait_expiry(30, None) == 0, _capi.last_error()
    assert lib.dvm_rt_sync(None) == -1
    msg = _capi.last_error()
    assert "bounded device wait expired" in msg and "vector 0x0f" in msg, msg
    assert lib.dvm_rt_check_status() == 0          # reading cleared it
    assert lib.dvm_rt_sync(None) == 0

    rng = np.random.default_rng(12)
    x = rng.standard_normal((300, 4096)).astype(np.float32)
    t = Tester("vector")
    s = t.store(t.sum(t.mul(t.load(x), 2.0), (1,), True))
    t.run()
    assert_close(t.output(s), (x * 2.0).sum(axis=1, keepdims=True), 1e-4, "launch after an expired wait")
    assert lib.dvm_rt_check_status() == 0
