"""``dvm.jit`` of the reference (python/dvm/jit.py) under its own import path."""
from dvm_b200.jit import JitKernel, kernel  # noqa: F401
