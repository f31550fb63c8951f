"""Import name of the reference package (python/dvm/__init__.py:17-42) for code written against it: ``import dvm``,
``dvm.kernel``, ``dvm.PyKernel``, ``from dvm.tester import Tester`` resolve to this repository's implementation
(``dvm_b200``), so the reference's examples and tests can be run unmodified with this repository's root on
``PYTHONPATH``."""
from dvm_b200 import *  # noqa: F401,F403
from dvm_b200 import __all__ as _names
from dvm_b200 import frontend as _core  # noqa: F401  (the reference exposes its extension module under this name)

__all__ = list(_names)
