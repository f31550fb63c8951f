"""``@kernel`` decorator: trace a Python function once into a fused-operator graph, then call it with NumPy
arrays.  Same contract as the reference's decorator (python/dvm/jit.py:20-78): the first parameter of the
decorated function is the kernel builder, the remaining ones are positional indices that ``load`` /
``scalar`` / ``int_array`` bind to call-time arguments; dynamic kernels re-run code generation on every
call with the shapes of the arrays passed in.
"""
import os

from .frontend import PyKernel


class JitKernel(PyKernel):
    def __init__(self, ker_type, dynamic):
        if dynamic:
            ker_type += ",dyn" if ":" in ker_type else ":dyn"
        dev_conf = os.getenv("DEVICE_ID")
        PyKernel.__init__(self, ker_type, "dev", int(dev_conf) if dev_conf else 0)
        self.inputs = None
        self.outputs = None
        self.dynamic = dynamic

    def build(self, func):
        nargs = func.__code__.co_argcount - 1
        self.inputs = [None] * nargs
        self.outputs = func(self, *range(nargs))
        if not self.dynamic:
            self.codegen(None)

    def load(self, index, dtype, shape=()):
        op = PyKernel.load(self, list(shape), dtype)
        self.inputs[index] = op
        return op

    def scalar(self, index):
        ref = PyKernel.scalar(self)
        self.inputs[index] = ref
        return ref

    def int_array(self, index):
        ref = PyKernel.int_array(self)
        self.inputs[index] = ref
        return ref

    def __call__(self, *args):
        for inp, arg in zip(self.inputs, args):
            PyKernel.input(self, inp, arg)
        if self.dynamic:
            self.codegen(None)
        self.run()
        if isinstance(self.outputs, (list, tuple)):
            return [self.output(x) for x in self.outputs]
        return self.output(self.outputs)


def kernel(ktype="split", dynamic=True):
    if callable(ktype):
        kobj = JitKernel("split", True)
        kobj.build(ktype)
        return kobj

    def decorate(func):
        kobj = JitKernel(ktype, dynamic)
        kobj.build(func)
        return kobj

    return decorate
