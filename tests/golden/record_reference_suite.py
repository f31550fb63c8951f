"""Records the reference's own unit tests for this path (mindspore-ai/dvm, tests/ut: every test marked `gpu`, plus the
unmarked MatMul / reduce / speculative-vector / tiling tests of the same files) as replayable fixtures.

The reference's tests build a graph through `dvm.tester.Tester`, feed NumPy inputs and compare the device result with a
NumPy expectation under a stated tolerance; they hold no stored vectors.  This script runs those test functions in THIS
container (where the reference tree is present) with `dvm` replaced by a recording Tester: every builder call, input
array, shape / scalar update, run and check is written down as an event, and nothing executes on a device.  The events
and arrays of every test that passes are saved to

    tests/golden/reference_suite.json      one entry per recorded test: its name and its events
    tests/golden/reference_suite.npz       the arrays the events refer to (inputs and expectations)

tests/test_reference_suite_gpu.py replays each entry on the GPU through this library's Tester and applies the recorded
checks.  A test whose arrays exceed the size cap is recorded without them ("spec" entries): each input is described by
its shape, dtype and value range, the replay draws seeded inputs from that description and the CPU oracle, evaluating
the same events, takes the place of the recorded expectation.  Tests that check through a Python callback or that use
builder methods this backend does not offer are left out and counted in the json header.

Usage (from the repository root; the reference tree is found as oracle/build_ref.py finds it):
    python -m tests.golden.record_reference_suite
"""
import json
import os
import sys
import types
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
CASE_CAP_BYTES = 96 * 1024       # arrays of one test
TOTAL_CAP_BYTES = 6 * 1024 * 1024
IN_SCOPE_FILES = ["test_matmul.py", "test_reduce.py", "test_spec_vector.py", "test_tiling.py", "test_reshape.py",
                  "test_broadcast.py", "test_unalign.py", "test_composite_ops.py", "test_dynamic_shape.py", "test_codegen.py"]
SPEC_CAP_BYTES = 96 * 1024 * 1024   # a test recorded without its arrays still has to replay in seconds


def spec_of(kind, a):
    """What the replay needs to draw a stand-in for input `a`."""
    d = {"shape": list(a.shape), "dtype": "bfloat16" if kind == "bf16" else a.dtype.name}
    v = a.astype(np.float32) if kind != "bf16" else (a.astype(np.uint32) << 16).view(np.float32)
    finite = v[np.isfinite(v)] if v.size else v
    d["lo"] = float(finite.min()) if finite.size else 0.0
    d["hi"] = float(finite.max()) if finite.size else 0.0
    d["integral"] = bool(a.dtype.kind in "iub" or (finite.size and np.all(finite == np.round(finite)) and d["hi"] - d["lo"] <= 4096))
    return d


def to_spec_events(events, arrays):
    """Events with every array replaced by its description; expectations are dropped (the oracle stands in)."""
    out = []
    for ev in events:
        if ev[0] == "call" and ev[2] in ("store_expect", "check") and len(ev[3]) >= 2:
            ev = ev[:3] + [[ev[3][0], None] + ev[3][2:]] + ev[4:]
        out.append(ev)

    def walk(v):
        if isinstance(v, dict) and "a" in v:
            kind, a = arrays[v["a"]]
            return {"spec": spec_of(kind, a)}
        if isinstance(v, dict) and "l" in v:
            return {"l": [walk(x) for x in v["l"]]}
        if isinstance(v, list):
            return [walk(x) for x in v]
        if isinstance(v, dict):
            return {k: walk(x) for k, x in v.items()}
        return v
    return [walk(ev) for ev in out]


class Trace:
    """Events of the test that is running."""

    def __init__(self):
        self.reset("")

    def reset(self, name):
        self.name = name
        self.events = []
        self.objects = []      # results of recorded calls (kept alive so that id() stays unique)
        self.index = {}        # id(object) -> position in `objects`
        self.arrays = []
        self.bad = None        # reason why the test cannot be recorded
        self.checks = 0

    def remember(self, obj):
        self.index[id(obj)] = len(self.objects)
        self.objects.append(obj)
        return len(self.objects) - 1

    def array(self, a):
        a = np.asarray(a)
        if str(a.dtype) == "bfloat16":
            self.arrays.append(("bf16", a.view(np.uint16)))
        else:
            self.arrays.append(("", a))
        return len(self.arrays) - 1

    def encode(self, v):
        from dvm_b200.frontend import DataType
        if id(v) in self.index:
            return {"o": self.index[id(v)]}
        if isinstance(v, RefProxy):
            return {"o": self.index[id(v)]}
        if isinstance(v, np.ndarray):
            return {"a": self.array(v)}
        if isinstance(v, DataType):
            return {"dt": int(v)}
        if isinstance(v, (bool, np.bool_)):
            return bool(v)
        if isinstance(v, (int, np.integer)):
            return int(v)
        if isinstance(v, (float, np.floating)):
            return float(v)
        if isinstance(v, str) or v is None:
            return v
        if isinstance(v, type) and issubclass(v, np.generic):
            return {"np": np.dtype(v).name}
        if isinstance(v, np.dtype):
            return {"np": v.name}
        if isinstance(v, (list, tuple)):
            return {"l": [self.encode(x) for x in v]}
        if callable(v):
            self.bad = "check through a Python callback"
            return None
        self.bad = "argument of type %s" % type(v).__name__
        return None


TRACE = Trace()


class RefProxy:
    """Stands for an IntArrayRef / ScalarRef handed to the test: updates are events."""

    def __init__(self, real):
        self._real = real

    def update(self, value):
        TRACE.events.append(["update", TRACE.index[id(self)], TRACE.encode(value)])
        self._real.update(value)

    def __getattr__(self, name):
        return getattr(self._real, name)


def make_recording_tester():
    from dvm_b200.frontend import IntArrayRef, NDObject, ScalarRef
    from dvm_b200.tester import Tester as RealTester

    class Tester:
        __test__ = False

        def __init__(self, ker_type="", use_pass_opt=False, run_mode="dev", comm=None):
            self._t = RealTester(ker_type, use_pass_opt, "das")   # compile only: nothing runs on a device here
            self._me = TRACE.remember(self)
            TRACE.events.append(["new", self._me, ker_type])

        @staticmethod
        def fast_random_normal(mean, std, shape):
            return np.random.normal(mean, std, shape)

        def __getattr__(self, name):
            return getattr(self._t, name)

    def unwrap(v):
        if isinstance(v, RefProxy):
            return v._real
        if isinstance(v, (list, tuple)):
            return type(v)(unwrap(x) for x in v)
        return v

    def wrap(name):
        def method(self, *args, **kwargs):
            enc_a = [TRACE.encode(a) for a in args]
            enc_k = {k: TRACE.encode(v) for k, v in kwargs.items()}
            real_args = [unwrap(a) for a in args]
            real_kw = {k: unwrap(v) for k, v in kwargs.items()}
            if name in ("run", "run_check", "check", "bare_run"):
                if name != "check":
                    self._t.codegen()
                if name in ("check", "run_check"):
                    TRACE.checks += 1
                TRACE.events.append(["call", self._me, name, enc_a, enc_k, None])
                return True
            if name in ("output", "perf", "run_perf", "msprof"):
                TRACE.bad = "the test reads device results itself (%s)" % name
                raise RuntimeError(TRACE.bad)
            out = getattr(self._t, name)(*real_args, **real_kw)
            res = None
            if isinstance(out, (IntArrayRef, ScalarRef)):
                out = RefProxy(out)
                res = TRACE.remember(out)
            elif isinstance(out, NDObject):
                res = TRACE.remember(out)
            TRACE.events.append(["call", self._me, name, enc_a, enc_k, res])
            return out
        method.__name__ = name
        return method

    for name in dir(RealTester):
        if not name.startswith("_") and not callable(getattr(RealTester, name)):
            setattr(Tester, name, getattr(RealTester, name))   # class constants the tests name (Tester.K_VEC, ...)
        if name.startswith("_") or not callable(getattr(RealTester, name)) or name in ("fast_random_normal",):
            continue
        if name in ("das", "dump", "dump_r", "inspect", "convert_to_bf16", "convert_from_bf16", "is_dynamic"):
            continue   # read-only helpers go straight to the real object
        setattr(Tester, name, wrap(name))
    return Tester


class Plugin:
    def __init__(self):
        self.cases = []
        self.arrays = {}
        self.skipped = {}
        self.total = 0

    def pytest_runtest_setup(self, item):
        np.random.seed(zlib.crc32(item.nodeid.encode()))
        TRACE.reset(item.nodeid)

    def pytest_runtest_logreport(self, report):
        if report.when != "call":
            return
        why = None
        if not report.passed:
            why = "not supported by this backend or failed while recording"
        elif TRACE.bad:
            why = TRACE.bad
        elif TRACE.checks == 0:
            why = "no Tester check in the test"
        nbytes = sum(a.nbytes for _, a in TRACE.arrays)
        if why is None and nbytes > CASE_CAP_BYTES:
            if nbytes <= SPEC_CAP_BYTES:
                self.cases.append({"name": TRACE.name, "spec": True, "events": to_spec_events(TRACE.events, TRACE.arrays)})
                return
            why = "arrays above the per-test cap"
        if why is None and self.total + nbytes > TOTAL_CAP_BYTES:
            why = "fixture file is full"
        if why is not None:
            self.skipped[why] = self.skipped.get(why, 0) + 1
            return
        base = len(self.arrays)
        kinds = []
        for i, (kind, a) in enumerate(TRACE.arrays):
            self.arrays["a%d" % (base + i)] = a
            kinds.append(kind)
        self.total += nbytes
        self.cases.append({"name": TRACE.name, "array_base": base, "array_kinds": kinds, "events": TRACE.events})


def main(ref=None):
    from oracle.build_ref import DEFAULT_REFERENCE
    ref = ref or DEFAULT_REFERENCE
    import pytest
    sys.path[:0] = [ROOT, ref]
    shim = types.ModuleType("dvm")
    import dvm_b200
    for n in dir(dvm_b200):
        setattr(shim, n, getattr(dvm_b200, n))
    tester_mod = types.ModuleType("dvm.tester")
    tester_mod.Tester = make_recording_tester()
    shim.tester = tester_mod
    shim.__path__ = []
    sys.modules["dvm"] = shim
    sys.modules["dvm.tester"] = tester_mod
    # the reference's tests import `tests.mark_utils.arg_mark` (platform / level marks): a pass-through stands in for it,
    # since `tests` already names this repository's own test package in this process
    marks = types.ModuleType("tests.mark_utils")
    marks.arg_mark = lambda **kw: (lambda fn: fn)
    sys.modules["tests.mark_utils"] = marks
    plugin = Plugin()
    os.chdir(ref)
    common = ["-q", "-p", "no:cacheprovider", "--no-header", "--continue-on-collection-errors"]
    pytest.main(["tests/ut", "-m", "gpu"] + common, plugins=[plugin])
    # the reference's CUDA backend has no MatMul and no max / min reduction, so its tests of those (and of the
    # speculative vector kernels and tilings on the same path) carry no gpu mark: take them from the files of this path
    pytest.main(["tests/ut/" + f for f in IN_SCOPE_FILES] + ["-m", "not gpu"] + common, plugins=[plugin])
    header = {"source": "mindspore-ai/dvm tests/ut: every test marked gpu, and the unmarked tests of " + ", ".join(IN_SCOPE_FILES),
              "recorded": len(plugin.cases),
              "with_arrays": sum(1 for c in plugin.cases if not c.get("spec")), "left_out": plugin.skipped}
    with open(os.path.join(HERE, "reference_suite.json"), "w") as f:
        json.dump({"header": header, "cases": plugin.cases}, f, separators=(",", ":"))
    np.savez_compressed(os.path.join(HERE, "reference_suite.npz"), **plugin.arrays)
    print(header, "arrays: %.1f KiB" % (plugin.total / 1024.0))


if __name__ == "__main__":
    main()
