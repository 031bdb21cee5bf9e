"""Compatibility alias of :mod:`aicomp_b200.parallel.schedule` under the reference's module name."""
from aicomp_b200.parallel.schedule import Schedule, ScheduleGPipe, Schedule1F1B, SCHEDULES  # noqa: F401
