"""``dvm.tester`` of the reference (python/dvm/tester.py) under its own import path."""
from dvm_b200.tester import *  # noqa: F401,F403
from dvm_b200.tester import Tester  # noqa: F401
