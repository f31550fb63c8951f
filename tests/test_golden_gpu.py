"""Device results against the committed golden vectors (tests/golden/oracle_golden.npz), through the C ABI: small
seeded instances of the five benchmark graphs under their tolerance classes and the integer / compare / select / cast
class bit for bit.  The oracle is not imported here: the fixtures are the target."""
import os

import numpy as np
import pytest

from tests.golden.make_golden import build, inputs
from tests.util import BF16, TOL_EXACT, TOL_FP32, TOL_HALF, TOL_REDUCE, assert_close

pytestmark = pytest.mark.gpu

KTYPE = {"c1": "vector", "c2": "vector", "c3": "vector:spec,dyn", "c4": "split", "c5": "mix", "exact": "vector"}
TOLS = {"c1": [TOL_FP32], "c2": [TOL_HALF, TOL_REDUCE, TOL_REDUCE], "c3": [TOL_HALF, TOL_HALF], "c4": [TOL_HALF],
        "c5": [TOL_HALF], "exact": [TOL_EXACT] * 8}


@pytest.mark.parametrize("name", sorted(KTYPE))
def test_against_golden(name):
    from dvm_b200.tester import Tester
    data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_golden.npz"))
    arrays, dts = inputs()[name]
    t = Tester(KTYPE[name])
    stores = [t.store(v) for v in build(name, t, [t.load(a, d) for a, d in zip(arrays, dts)])]
    t.run()
    for i, (s, tol) in enumerate(zip(stores, TOLS[name])):
        want = data["%s_%d" % (name, i)]
        got = t.output(s)
        if BF16 is not None and got.dtype == BF16:
            want = want.view(BF16)
        assert_close(got, want, tol, "%s output %d" % (name, i))
