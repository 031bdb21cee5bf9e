"""tcgen05 flash attention (forward/backward) bindings."""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib


def supported(qkv: torch.Tensor, head_dim: int) -> bool:
    """True when the sm_100a flash-attention kernels serve this call."""
    if not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim == 128):
        return False
    lib = _lib.require()
    return hasattr(lib, "b200_flash_fwd") and _ENABLED


_ENABLED = False


def flash_attention_packed(qkv, B, S, hq, hkv, D, scale: Optional[float] = None):
    raise NotImplementedError
