"""Replays the reference's own GPU-marked unit tests on the device.

tests/golden/reference_suite.{json,npz} hold, for each recorded test of mindspore-ai/dvm's tests/ut (`-m gpu`), the
sequence of Tester calls it makes, its input arrays and the NumPy expectations it computes, as written down by
tests/golden/record_reference_suite.py while running the reference's test functions.  Each entry is replayed here through
this library's Tester on the GPU, and every check of the original test (`run_check`, `check`) must hold under the tolerance
the original test states (the Tester defaults otherwise: 1e-5 fp32, 1e-3 fp16, exact for the rest).
"""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))

with open(os.path.join(HERE, "golden", "reference_suite.json")) as f:
    SUITE = json.load(f)
CASES = SUITE["cases"]
_ARRAYS = None


def arrays():
    global _ARRAYS
    if _ARRAYS is None:
        _ARRAYS = np.load(os.path.join(HERE, "golden", "reference_suite.npz"))
    return _ARRAYS


def decode(v, case, objects):
    if isinstance(v, dict):
        if "o" in v:
            return objects[v["o"]]
        if "a" in v:
            a = arrays()["a%d" % (case["array_base"] + v["a"])]
            if case["array_kinds"][v["a"]] == "bf16":
                import ml_dtypes
                a = a.view(ml_dtypes.bfloat16)
            return a
        if "dt" in v:
            from dvm_b200.frontend import DataType
            return DataType(v["dt"])
        if "np" in v:
            return np.dtype(v["np"]).type
        if "l" in v:
            return [decode(x, case, objects) for x in v["l"]]
    return v


def replay(case):
    from dvm_b200.tester import Tester
    objects = {}
    for ev in case["events"]:
        if ev[0] == "new":
            objects[ev[1]] = Tester(ev[2])
        elif ev[0] == "update":
            objects[ev[1]].update(decode(ev[2], case, objects))
        else:
            _, who, name, args, kwargs, res = ev
            out = getattr(objects[who], name)(*[decode(a, case, objects) for a in args],
                                              **{k: decode(v, case, objects) for k, v in kwargs.items()})
            if name in ("run_check", "check"):
                assert out, "%s: %s failed" % (case["name"], name)
            if res is not None:
                objects[res] = out


def test_the_fixture_covers_the_reference_suite():
    assert SUITE["header"]["recorded"] == len(CASES) and len(CASES) >= 200


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=[c["name"].split("/")[-1] for c in CASES])
def test_reference_test_replayed(case):
    replay(case)
