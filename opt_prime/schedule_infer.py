"""Compatibility alias of :mod:`aicomp_b200.parallel.schedule_infer` under the reference's module name."""
from aicomp_b200.parallel.schedule_infer import ScheduleInference, ScheduleGeneration  # noqa: F401
