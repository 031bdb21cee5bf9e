"""Attention entry points.

``causal_attention_packed`` consumes the packed QKV projection
``[tokens, (Hq + 2 Hkv) * D]`` directly (GQA native: no ``repeat_kv``) and
returns ``[tokens, Hq * D]`` ready for the output projection.  On B200 with
bf16 inputs it runs the tcgen05 flash-attention kernels of this library; the
PyTorch expression below is the CPU / fp32 path and the test oracle.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


__all__ = ["causal_attention_packed", "attention_reference"]


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, scale: Optional[float] = None,
                        q_offset: int = 0) -> torch.Tensor:
    """fp32 softmax(QK^T)V for ``q [B,Hq,Sq,D]``, ``k/v [B,Hkv,Sk,D]`` (GQA by head grouping)."""
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().view(B, Hkv, g, Sq, D)
    s = torch.einsum("bhgqd,bhkd->bhgqk", qf, k.float()) * scale
    if causal:
        qi = torch.arange(Sq, device=q.device)[:, None] + q_offset
        ki = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(ki > qi, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhgqk,bhkd->bhgqd", p, v.float())
    return o.reshape(B, Hq, Sq, D).to(q.dtype)


def _split_packed(qkv: torch.Tensor, B: int, S: int, hq: int, hkv: int, D: int):
    q = qkv[:, : hq * D].view(B, S, hq, D).transpose(1, 2)
    k = qkv[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D).transpose(1, 2)
    v = qkv[:, (hq + hkv) * D:].view(B, S, hkv, D).transpose(1, 2)
    return q, k, v


def causal_attention_packed(qkv: torch.Tensor, B: int, S: int, hq: int, hkv: int, D: int, scale: Optional[float] = None
                            ) -> torch.Tensor:
    from . import flash
    if qkv.is_cuda and flash.supported(qkv, D):
        return flash.flash_attention_packed(qkv, B, S, hq, hkv, D, scale)
    q, k, v = _split_packed(qkv, B, S, hq, hkv, D)
    if qkv.is_cuda:
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale, enable_gqa=(hq != hkv))
    else:
        o = attention_reference(q, k, v, True, scale)
    return o.transpose(1, 2).reshape(B * S, hq * D)
