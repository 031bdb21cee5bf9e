"""tcgen05 flash-attention bindings (forward kernel; backward through the recompute path below)."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib

_lib.OPTIONAL_PROTOS.update({
    "b200_flash_fwd": [_lib.P, _lib.L, _lib.P, _lib.L, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.I, _lib.F, _lib.I, _lib.P, _lib.P],
})
_lib.rebind()

# Training keeps the library attention until the backward kernel of this framework is enabled; inference
# (no autograd) always runs the forward kernel.
TRAINING_USES_KERNEL = False


def supported(qkv: torch.Tensor, head_dim: int) -> bool:
    """True when the sm_100a flash-attention forward kernel serves this call."""
    if not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim == 128 and qkv.stride(-1) == 1):
        return False
    lib = _lib.require()
    if not hasattr(lib, "b200_flash_fwd"):
        return False
    if torch.is_grad_enabled() and qkv.requires_grad and not TRAINING_USES_KERNEL:
        return False
    return True


def flash_fwd(qkv: torch.Tensor, B: int, S: int, hq: int, hkv: int, D: int, scale: Optional[float] = None, causal: bool = True,
              need_lse: bool = False):
    from . import _count
    lib = _lib.require()
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty(B * S, hq * D, dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty(B, hq, S, dtype=torch.float32, device=qkv.device) if need_lse else None
    rc = lib.b200_flash_fwd(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), _lib.ptr(lse), B, S, hq, hkv, D,
                            float(scale), int(causal), _lib.err_word(qkv.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "flash_fwd")
    _count()
    return out, lse


def flash_attention_packed(qkv, B, S, hq, hkv, D, scale: Optional[float] = None):
    out, _ = flash_fwd(qkv, B, S, hq, hkv, D, scale, True, False)
    return out
