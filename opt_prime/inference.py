"""Compatibility alias of :mod:`aicomp_b200.inference` under the reference's module name."""
from aicomp_b200.inference import Optimus_Inference, sample_token  # noqa: F401
