"""Adapter over the reference's own `_dvm_py` module (built by oracle/build_ref.py into oracle/_ref/) so that the
graph definitions of the parity tests can be evaluated by the reference's CUDA backend on the same GPU.
Test and benchmark-baseline infrastructure only: nothing in the product imports it."""
import glob
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_NAMES = ["bool", "float16", "bfloat16", "float32", "int32", "int64"]
_module = None


def module():
    """The reference extension module, or None when it was not built."""
    global _module
    if _module is None:
        hits = glob.glob(os.path.join(ROOT, "oracle", "_ref", "_dvm_py*.so"))
        if not hits:
            return None
        spec = importlib.util.spec_from_file_location("_dvm_py", hits[0])
        _module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_module)
    return _module


class RefKernel:
    """Same surface as dvm_b200.tester.Tester for what the shared graph definitions use."""

    def __init__(self, ker_type="vector"):
        self.m = module()
        self.k = self.m.PyKernel(ker_type, "dev", int(os.environ.get("DEVICE_ID", "0")))
        self._stores = []
        self._inputs = []   # (load op, host array in the form the reference's input() takes)

    def _dt(self, code):
        return getattr(self.m.DataType, _NAMES[int(code)])

    def load(self, array, dtype=None):
        array = np.ascontiguousarray(array)
        if dtype is None and str(array.dtype) == "bfloat16":
            code = 2
        elif dtype is None:
            code = {np.dtype(np.bool_): 0, np.dtype(np.float16): 1, np.dtype(np.float32): 3, np.dtype(np.int32): 4}[array.dtype]
        else:
            code = int(dtype)
        if code == 2 and array.dtype == np.float32:
            array = self.k.convert_to_bf16(array)
        elif code == 2:
            array = array.view(np.uint16)   # the reference moves bf16 as raw 16-bit words
        elif code == 1:
            array = array.astype(np.float16)
        op = self.k.load(list(array.shape), self._dt(code))
        self.k.input(op, array)
        self._inputs.append((op, array))
        return op

    def cast(self, x, dtype):
        return self.k.cast(x, self._dt(dtype))

    def full(self, scalar, shape, dtype):
        return self.k.full(scalar, list(shape), self._dt(dtype))

    def store(self, x):
        s = self.k.store(x)
        self._stores.append(s)
        return s

    def run(self):
        self.k.codegen(None)
        self.k.run()

    def output(self, s, bf16=False):
        out = self.k.output(s)
        return self.k.convert_from_bf16(out) if bf16 else out

    def perf(self):
        return self.k.perf()

    def step_from_host(self):
        """One step of the reference's own host-buffer path: input() of every load (its device allocation and
        synchronous upload, src/pybind_api.cc:217-223, 819-842), run() (launch and stream wait, :689-701) and output()
        of every store (download, :856-865).  Returns (bytes uploaded, bytes downloaded)."""
        up = down = 0
        for op, array in self._inputs:
            self.k.input(op, array)
            up += array.nbytes
        self.k.run()
        for s in self._stores:
            down += self.k.output(s).nbytes
        return up, down

    def __getattr__(self, name):   # every other builder method goes straight to the reference
        return getattr(self.k, name)
