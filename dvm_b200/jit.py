"""``@kernel``: turn a Python function that describes a fused-operator graph into a callable on NumPy arrays.

The contract is the reference decorator's (python/dvm/jit.py): the decorated function receives the kernel builder as
its first argument; each further parameter stands for one call-time argument, and the function binds it by passing it
to ``load(param, dtype[, shape])``, ``scalar(param)`` or ``int_array(param)``.  What the function returns (one store or
a list / tuple of stores) is what a call returns.  ``@kernel`` alone means a dynamic-shape "split" kernel, which
re-plans for the shapes of the arrays of every call; ``@kernel(ktype, dynamic=False)`` plans once, at decoration, for
the shapes given to ``load``.

The implementation is this package's own: the graph is traced once with placeholder objects (one ``_Slot`` per
parameter) over a ``PyKernel`` that the wrapper owns; a call feeds the slots in order, plans if the kernel is dynamic,
runs and downloads.
"""
import inspect
import os

from .frontend import PyKernel


class _Slot:
    """Placeholder for the call-time argument at `position`; remembers what the trace bound it to."""
    __slots__ = ("position", "name", "target")

    def __init__(self, position, name):
        self.position, self.name, self.target = position, name, None


def _kernel_type_string(ktype, dynamic):
    if not dynamic:
        return ktype
    head, sep, flags = ktype.partition(":")
    names = [f for f in flags.split(",") if f] if sep else []
    if "dyn" not in names:
        names.append("dyn")
    return head + ":" + ",".join(names)


class JitKernel:
    """A traced graph plus its runner.  Builder methods that the traced function calls and that are not overridden here
    (add, mul, sum, store, ...) are the underlying PyKernel's."""

    def __init__(self, ker_type, dynamic):
        device = os.getenv("DEVICE_ID")
        self._runner = PyKernel(_kernel_type_string(ker_type, dynamic), "dev", int(device) if device else 0)
        self.dynamic = bool(dynamic)
        self._slots = []
        self._results = None
        self._static_loads = []

    # -- tracing
    def build(self, func):
        params = list(inspect.signature(func).parameters)[1:]
        self._slots = [_Slot(i, name) for i, name in enumerate(params)]
        self._results = func(self, *self._slots)
        if not self.dynamic:
            # a static kernel is planned here, once: its loads get device buffers of their declared shapes now and every
            # call copies into them
            import numpy as np
            from .frontend import np_dtype_of
            for op, shape, dtype in self._static_loads:
                self._runner.input(op, np.zeros(shape, np_dtype_of(dtype)))
            self._runner.codegen(None)
        return self

    def _bind(self, slot, target):
        if not isinstance(slot, _Slot):
            raise TypeError("the first argument of load / scalar / int_array must be one of the kernel function's parameters")
        slot.target = target
        return target

    def load(self, slot, dtype, shape=()):
        op = self._bind(slot, self._runner.load(list(shape), dtype))
        self._static_loads.append((op, tuple(shape), dtype))
        return op

    def scalar(self, slot):
        return self._bind(slot, self._runner.scalar())

    def int_array(self, slot):
        return self._bind(slot, self._runner.int_array())

    def __getattr__(self, name):
        return getattr(self._runner, name)

    # -- calling
    def __call__(self, *args):
        if len(args) != len(self._slots):
            raise TypeError("this kernel takes %d arguments (%d given)" % (len(self._slots), len(args)))
        for slot, value in zip(self._slots, args):
            if slot.target is not None:      # a parameter the function never bound is ignored
                self._runner.input(slot.target, value)
        if self.dynamic:
            self._runner.codegen(None)
        self._runner.run()
        if isinstance(self._results, (list, tuple)):
            return [self._runner.output(s) for s in self._results]
        return self._runner.output(self._results)


def kernel(ktype="split", dynamic=True):
    """Decorator, usable bare (``@kernel``) or with arguments (``@kernel("vector", dynamic=False)``)."""
    if callable(ktype):
        return JitKernel("split", True).build(ktype)
    return lambda func: JitKernel(ktype, dynamic).build(func)
