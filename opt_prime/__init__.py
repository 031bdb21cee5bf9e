"""Drop-in ``opt_prime`` namespace: scripts written for OptimusPrime import from here and run on aicomp_b200.

``from opt_prime.opti_pri import Optimus_p`` / ``from opt_prime.inference import Optimus_Inference`` /
``from opt_prime.lora import LoRAConfig`` / ``from opt_prime.IR import IR_Anal`` keep working.  Names resolve
lazily (PEP 562) so ``opt_prime.mps_manager`` can be imported before ``torch``, as in the reference
(opt_prime/opt_prime/__init__.py:27-37).
"""
import importlib

_LAZY = {"Optimus_p": "aicomp_b200.engine", "IR_Anal": "aicomp_b200.engine", "Optimus_Inference": "aicomp_b200.inference",
         "LoRAConfig": "aicomp_b200.lora", "KVCacheManager": "aicomp_b200.kv_cache",
         "CachedScaledDotProductAttention": "aicomp_b200.kv_cache"}
__all__ = list(_LAZY)


def __getattr__(name):
    if name in _LAZY:
        return getattr(importlib.import_module(_LAZY[name]), name)
    raise AttributeError(f"module 'opt_prime' has no attribute {name!r}")
