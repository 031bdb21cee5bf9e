"""Compatibility alias of :mod:`aicomp_b200.utils.mps_manager` under the reference's module name."""
from aicomp_b200.utils.mps_manager import resolve_visible_devices, restore_visible_devices, setup_mps_for_inference, MPSManager, FileBarrier  # noqa: F401
