"""Compatibility alias of :mod:`aicomp_b200.kv_cache` under the reference's module name."""
from aicomp_b200.kv_cache import KVCacheManager, CachedScaledDotProductAttention, DenseKVAdaptor  # noqa: F401
