"""aicomp_b200: Blackwell-native automatic PP x TP x DP training and serving framework.

Names are resolved lazily (PEP 562) so that light-weight submodules such as
``aicomp_b200.utils.mps_manager`` can be imported before ``torch`` (the reference
package does the same, opt_prime/opt_prime/__init__.py:27-37).
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_LAZY = {
    "Optimus_p": ("aicomp_b200.engine", "Optimus_p"),
    "IR_Anal": ("aicomp_b200.engine", "IR_Anal"),
    "Optimus_Inference": ("aicomp_b200.inference", "Optimus_Inference"),
    "LoRAConfig": ("aicomp_b200.lora", "LoRAConfig"),
    "KVCacheManager": ("aicomp_b200.kv_cache", "KVCacheManager"),
    "FusedAdamW": ("aicomp_b200.optim.adamw", "FusedAdamW"),
}

__all__ = list(_LAZY) + ["__version__"]


def __getattr__(name: str):
    if name in _LAZY:
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module 'aicomp_b200' has no attribute {name!r}")
