"""dvm_b200: B200-native device virtual machine for fused tensor operators.

Drop-in for the fused-operator path of mindspore-ai/dvm: the package exports the names of the reference's
``dvm`` Python package (python/dvm/__init__.py:17-42) - DataType, Device, Kernel, PyKernel, NDObject,
IntArrayRef, ScalarRef, the dtype aliases and the ``kernel`` decorator - implemented over the C ABI of
``libdvm_b200.so`` (include/dvm_c.h).
"""
from .frontend import DataType, Device, Kernel, PyKernel, NDObject, IntArrayRef, ScalarRef, DvmError
from .jit import kernel, JitKernel

bool_ = DataType.bool
float16 = DataType.float16
bfloat16 = DataType.bfloat16
float32 = DataType.float32
int32 = DataType.int32
int64 = DataType.int64

__all__ = [
    "DataType", "Device", "Kernel", "PyKernel", "NDObject", "IntArrayRef", "ScalarRef", "DvmError",
    "kernel", "JitKernel", "bool_", "float16", "bfloat16", "float32", "int32", "int64",
]
