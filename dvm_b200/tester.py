"""Test harness over PyKernel, with the surface of the reference's Tester (python/dvm/tester.py:70-299):
``load`` takes a NumPy array (uploading it) or a shape for dynamic kernels, ``store_expect`` records an
expectation, ``run_check`` runs and compares with ``np.allclose(rtol=eps, atol=eps, equal_nan=True)`` using
the reference's default tolerances (1e-5 fp32, 1e-3 fp16, 0 otherwise).
"""
import inspect
import os

import numpy as np

from .frontend import DataType, PyKernel, dvm_dtype_of, _BF16


def _normalize_dtype(dtype):
    if isinstance(dtype, DataType):
        return dtype
    if isinstance(dtype, (int, np.integer)) and not isinstance(dtype, bool):
        return DataType(int(dtype))
    if isinstance(dtype, str):
        names = {"bool": DataType.bool, "float16": DataType.float16, "bfloat16": DataType.bfloat16,
                 "float32": DataType.float32, "int32": DataType.int32, "int64": DataType.int64}
        return names[dtype]
    return dvm_dtype_of(dtype)


class Tester(PyKernel):
    __test__ = False

    def __init__(self, ker_type="", use_pass_opt=False, run_mode="dev"):
        dev_conf = os.getenv("DEVICE_ID")
        PyKernel.__init__(self, ker_type, run_mode, int(dev_conf) if dev_conf else 0)
        self.is_dyn = "dyn" in ker_type
        self.is_codegen = False
        self.expects = []  # [store op, expectation, eps]

    @staticmethod
    def fast_random_normal(mean, std, shape):
        """Normal samples of `shape` (python/dvm/tester.py: a faster stand-in for np.random.normal on large shapes)."""
        return np.random.default_rng().standard_normal(tuple(shape), dtype=np.float32) * np.float32(std) + np.float32(mean)

    @staticmethod
    def bf16_random_normal(loc, scale, shape):
        """fp32 normal samples whose values are exactly representable in bfloat16 (python/dvm/tester.py:93-99)."""
        x = np.random.normal(loc, scale, shape).astype(np.float32)
        return (x.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)

    def load(self, shape_arr, dtype=None):
        if not isinstance(shape_arr, np.ndarray):
            return PyKernel.load(self, shape_arr, _normalize_dtype(dtype))   # dynamic-shape declaration
        dtype_id = _normalize_dtype(shape_arr.dtype if dtype is None else dtype)
        if dtype_id == DataType.bfloat16 and (_BF16 is None or shape_arr.dtype != _BF16):
            shape_arr = PyKernel.convert_to_bf16(shape_arr)
        elif dtype_id == DataType.float16 and shape_arr.dtype != np.float16:
            shape_arr = shape_arr.astype(np.float16)
        elif dtype_id == DataType.float32 and shape_arr.dtype != np.float32:
            shape_arr = shape_arr.astype(np.float32)
        op = PyKernel.load(self, list(shape_arr.shape), dtype_id)
        self.input(op, shape_arr)
        return op

    def _whole_array(self, arr, dtype):
        dtype_id = _normalize_dtype(arr.dtype if dtype is None else dtype)
        if dtype_id == DataType.bfloat16 and (_BF16 is None or arr.dtype != _BF16):
            arr = PyKernel.convert_to_bf16(arr)
        return arr, dtype_id

    def slice_load(self, shape_arr, start, size, dtype=None):
        """python/dvm/tester.py:151-160: the window start + size of an array (or of a dynamic-shape input)."""
        if not isinstance(shape_arr, np.ndarray):
            return PyKernel.slice_load(self, shape_arr, start, size, _normalize_dtype(dtype))
        arr, dtype_id = self._whole_array(shape_arr, dtype)
        op = PyKernel.slice_load(self, list(arr.shape), start, size, dtype_id)
        self.input(op, arr)
        return op

    def stridedslice_load(self, shape_arr, start, end, step, dtype=None):
        """python/dvm/tester.py:162-171: the window start / end / step of an array, read as Python slices are."""
        if not isinstance(shape_arr, np.ndarray):
            return PyKernel.stridedslice_load(self, shape_arr, start, end, step, _normalize_dtype(dtype))
        arr, dtype_id = self._whole_array(shape_arr, dtype)
        op = PyKernel.stridedslice_load(self, list(arr.shape), start, end, step, dtype_id)
        self.input(op, arr)
        return op

    def view_load(self, shape, stride, arr_dtype, offset=0, real_dtype=None):
        """python/dvm/tester.py:120-132: a strided window of an array (or, given a dtype, of a dynamic-shape input)."""
        if not isinstance(arr_dtype, np.ndarray):
            return PyKernel.view_load(self, shape, stride, _normalize_dtype(arr_dtype))
        arr = arr_dtype
        dtype_id = _normalize_dtype(arr.dtype)
        if real_dtype is not None:
            dtype_id = _normalize_dtype(real_dtype)
            if dtype_id == DataType.bfloat16:
                arr = PyKernel.convert_to_bf16(arr)
        op = PyKernel.view_load(self, shape, stride, dtype_id)
        self.input(op, arr, offset)
        return op

    def view_store_expect(self, x, stride, e, eps=None):
        """python/dvm/tester.py:205-209: a strided store into a zero-filled buffer of the expectation's size."""
        op = PyKernel.view_store(self, x, stride)
        self.expects.append([op, e, eps])
        self.set_output(op, np.ascontiguousarray(np.zeros_like(e)))
        return op

    def cast(self, x, dtype):
        return PyKernel.cast(self, x, _normalize_dtype(dtype))

    def full(self, scalar, shape, dtype=None):
        return PyKernel.full(self, scalar, shape, _normalize_dtype(dtype))

    def store_expect(self, x, e, eps=None):
        op = PyKernel.store(self, x)
        self.expects.append([op, e, eps])
        return op

    def codegen(self, verbose=False):
        if self.is_codegen:
            return
        PyKernel.codegen(self, None)
        if verbose:
            print(self.dump_r())
            print(self.das())
        if not self.is_dyn:
            self.is_codegen = True

    def run(self, verbose=False):
        self.codegen(verbose)
        PyKernel.run(self)

    def bare_run(self):
        PyKernel.run(self)

    def check(self, store, expect, eps=None, verbose=False):
        out = self.output(store)
        if store.dtype() == DataType.bfloat16:
            out = PyKernel.convert_from_bf16(out)
        if inspect.isfunction(expect):
            return bool(expect(out))
        if eps is None:
            eps = 1e-5 if out.dtype == np.float32 else (1e-3 if out.dtype == np.float16 else 0)
        expect = np.asarray(expect)
        if _BF16 is not None and expect.dtype == _BF16:
            expect = expect.astype(np.float32)
        ok = np.allclose(out, expect, rtol=eps, atol=eps, equal_nan=True)
        if not ok and verbose:
            bad = ~np.isclose(out, expect, rtol=eps, atol=eps, equal_nan=True)
            idx = np.argwhere(bad)[:8]
            for i in idx:
                print("mismatch at", tuple(i), "expect", expect[tuple(i)], "got", out[tuple(i)])
        return bool(ok)

    def run_check(self, verbose=False):
        self.run(verbose)
        return all(self.check(op, e, eps, verbose) for op, e, eps in self.expects)

    def reset(self):
        PyKernel.reset(self)
        self.is_codegen = False
        self.expects = []

    def run_perf(self):
        self.codegen()
        return self.perf()
