"""Compatibility alias: ``IR`` and ``IR_Anal`` under the reference's module name."""
from aicomp_b200.engine import IR_Anal  # noqa: F401
from aicomp_b200.graph.ir import IR  # noqa: F401
