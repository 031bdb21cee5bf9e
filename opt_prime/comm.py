"""Compatibility alias of :mod:`aicomp_b200.parallel.comm` under the reference's module name."""
from aicomp_b200.parallel.comm import Comm, Channel  # noqa: F401
