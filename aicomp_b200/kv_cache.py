"""Dense KV cache for the static-batch inference engine.

API parity with the reference (opt_prime/opt_prime/kv_cache.py:19-424): ``KVCacheManager`` pre-allocates
``[B, max_seq_len, kv_heads, head_dim]`` K and V per layer and hands out prefix views; one shared sequence
length covers all layers.  ``CachedScaledDotProductAttention`` is a drop-in module for the
``scaled_dot_product_attention`` call of a traced graph (generic models).  Differences: the cache stores
the GQA key/value heads (8 for Llama-3-8B), not the 32 repeated heads the reference caches
(examples/pp_generation_llama.py:247-251), and decode batches keep their ``[B, 1]`` shape.
The paged, per-sequence cache used for serving lives in :mod:`aicomp_b200.serve.paged_kv`.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .ops import attention as attn_ops

__all__ = ["KVCacheManager", "CachedScaledDotProductAttention", "DenseKVAdaptor"]


class KVCacheManager:
    def __init__(self, num_layers: int, num_heads: int, head_dim: int, max_batch_size: int = 32, max_seq_len: int = 2048,
                 dtype: torch.dtype = torch.bfloat16, device=None, layer_offset: int = 0):
        self.num_layers, self.num_heads, self.head_dim = num_layers, num_heads, head_dim
        self.max_batch_size, self.max_seq_len = max_batch_size, max_seq_len
        self.dtype, self.device = dtype, device
        self.layer_offset = layer_offset
        self._cache: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._seq_len = 0
        self._batch = 0

    def allocate(self, batch_size: Optional[int] = None) -> None:
        b = batch_size or self.max_batch_size
        if b > self.max_batch_size:
            raise ValueError(f"batch {b} exceeds max_batch_size {self.max_batch_size}")
        self._batch = b
        for l in range(self.num_layers):
            shape = (b, self.max_seq_len, self.num_heads, self.head_dim)
            self._cache[l] = (torch.zeros(shape, dtype=self.dtype, device=self.device),
                              torch.zeros(shape, dtype=self.dtype, device=self.device))
        self._seq_len = 0

    @property
    def is_allocated(self) -> bool:
        return bool(self._cache)

    @property
    def seq_len(self) -> int:
        return self._seq_len

    def update(self, layer: int, k: torch.Tensor, v: torch.Tensor, position: Optional[int] = None):
        """Write ``k, v [B, S, heads, D]`` at ``position`` (default: append) and return the valid prefixes."""
        l = layer - self.layer_offset
        if l not in self._cache:
            raise KeyError(f"layer {layer} has no cache on this stage")
        ck, cv = self._cache[l]
        start = self._seq_len if position is None else position
        S, B = k.shape[1], k.shape[0]
        if start + S > self.max_seq_len:
            raise ValueError(f"sequence {start + S} exceeds max_seq_len {self.max_seq_len}")
        ck[:B, start:start + S] = k
        cv[:B, start:start + S] = v
        return ck[:B, :start + S], cv[:B, :start + S]

    def advance(self, n: int) -> None:
        self._seq_len += n

    def clear(self) -> None:
        self._seq_len = 0

    def free(self) -> None:
        self._cache.clear()
        self._seq_len = 0

    def memory_bytes(self) -> int:
        return sum(k.numel() * k.element_size() * 2 for k, _ in self._cache.values())


def _attend_with_prefix(q, k_all, v_all, start: int, scale: Optional[float]):
    """q [B,S,Hq,D] at absolute positions start..start+S-1 over k_all/v_all [B,start+S,Hkv,D]."""
    qh, kh, vh = q.transpose(1, 2), k_all.transpose(1, 2), v_all.transpose(1, 2)
    if q.is_cuda:
        S, T = q.shape[1], k_all.shape[1]
        if S == 1:
            o = F.scaled_dot_product_attention(qh, kh, vh, is_causal=False, scale=scale, enable_gqa=qh.shape[1] != kh.shape[1])
        else:
            mask = torch.ones(S, T, dtype=torch.bool, device=q.device).tril(T - S)
            o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, scale=scale, enable_gqa=qh.shape[1] != kh.shape[1])
    else:
        o = attn_ops.attention_reference(qh, kh, vh, causal=True, scale=scale, q_offset=start)
    return o.transpose(1, 2)


class DenseKVAdaptor:
    """Connects fused Llama layers to a :class:`KVCacheManager` (``layer.kv_cache = adaptor``)."""

    def __init__(self, manager: KVCacheManager):
        self.m = manager
        self.enabled = True

    def attend(self, layer, qkv: torch.Tensor, B: int, S: int, pos: torch.Tensor) -> torch.Tensor:
        hq, hkv, D = layer.hq, layer.hkv, layer.head_dim
        if not self.enabled:
            return attn_ops.causal_attention_packed(qkv, B, S, hq, hkv, D)
        q = qkv[:, : hq * D].view(B, S, hq, D)
        k = qkv[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D)
        v = qkv[:, (hq + hkv) * D:].view(B, S, hkv, D)
        start = self.m.seq_len
        k_all, v_all = self.m.update(layer.layer_idx, k, v, start)
        if start == 0:
            return attn_ops.causal_attention_packed(qkv, B, S, hq, hkv, D)
        o = _attend_with_prefix(q, k_all, v_all, start, None)
        return o.reshape(B * S, hq * D)


class CachedScaledDotProductAttention(nn.Module):
    """Module form of ``F.scaled_dot_product_attention`` with an incremental KV cache.

    Swapped into a traced graph in place of the SDPA ``call_function`` (generic, non-fused models).
    Prefill ignores the traced mask and runs causal attention; decode attends the new tokens over the
    cached prefix.  Uses an external :class:`KVCacheManager` when attached, else an internal cache.
    """

    def __init__(self, layer_idx: int, max_batch_size: int = 32, max_seq_len: int = 2048):
        super().__init__()
        self.layer_idx = layer_idx
        self.max_batch_size, self.max_seq_len = max_batch_size, max_seq_len
        self.enabled = False
        self.manager: Optional[KVCacheManager] = None
        self._k = self._v = None
        self._len = 0

    def enable(self) -> None:
        self.enabled = True

    def disable(self) -> None:
        self.enabled = False

    def attach(self, manager: KVCacheManager) -> None:
        self.manager = manager

    def clear(self) -> None:
        self._len = 0

    def free(self) -> None:
        self._k = self._v = None
        self._len = 0

    def forward(self, query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False):
        if not self.enabled:
            return F.scaled_dot_product_attention(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal,
                                                  scale=scale, enable_gqa=enable_gqa)
        B, H, S, D = key.shape
        k_new, v_new = key.transpose(1, 2), value.transpose(1, 2)  # [B,S,H,D]
        if self.manager is not None:
            start = self.manager.seq_len
            k_all, v_all = self.manager.update(self.layer_idx, k_new, v_new, start)
        else:
            if self._k is None or self._k.shape[0] < B:
                shape = (max(B, 1), self.max_seq_len, H, D)
                self._k = torch.zeros(shape, dtype=key.dtype, device=key.device)
                self._v = torch.zeros(shape, dtype=key.dtype, device=key.device)
                self._len = 0
            start = self._len
            self._k[:B, start:start + S] = k_new
            self._v[:B, start:start + S] = v_new
            self._len = start + S
            k_all, v_all = self._k[:B, :start + S], self._v[:B, :start + S]
        o = _attend_with_prefix(query.transpose(1, 2), k_all, v_all, start, scale)
        return o.transpose(1, 2)
