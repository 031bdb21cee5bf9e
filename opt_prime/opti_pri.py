"""Compatibility alias of :mod:`aicomp_b200.engine` under the reference's module name."""
from aicomp_b200.engine import Optimus_p, IR_Anal  # noqa: F401
