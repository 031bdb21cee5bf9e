"""tcgen05 flash-attention bindings: forward and backward kernels on the packed QKV projection."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib

_lib.OPTIONAL_PROTOS.update({
    "b200_flash_fwd": [_lib.P, _lib.L, _lib.P, _lib.L, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I, _lib.I, _lib.F, _lib.I, _lib.P, _lib.P],
    "b200_flash_bwd": [_lib.P, _lib.L, _lib.P, _lib.L, _lib.P, _lib.L, _lib.P, _lib.P, _lib.P, _lib.P, _lib.I, _lib.I, _lib.I, _lib.I,
                       _lib.I, _lib.F, _lib.I, _lib.P, _lib.P],
})
_lib.rebind()

# Training runs the forward and backward kernels of this library; set to False to fall back to the library
# attention (cuDNN SDPA) for an A/B comparison.
TRAINING_USES_KERNEL = True


def supported(qkv: torch.Tensor, head_dim: int) -> bool:
    """True when the sm_100a flash-attention forward kernel serves this call."""
    if not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim == 128 and qkv.stride(-1) == 1):
        return False
    lib = _lib.require()
    if not hasattr(lib, "b200_flash_fwd"):
        return False
    if torch.is_grad_enabled() and qkv.requires_grad and not (TRAINING_USES_KERNEL and hasattr(lib, "b200_flash_bwd")):
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


def flash_bwd(qkv: torch.Tensor, out: torch.Tensor, dout: torch.Tensor, lse: torch.Tensor, B: int, S: int, hq: int, hkv: int, D: int,
              scale: Optional[float] = None, causal: bool = True) -> torch.Tensor:
    """Gradient of the packed QKV projection, [B*S, (hq + 2 hkv) * D] bf16, from dO [B*S, hq*D]."""
    from . import _count
    lib = _lib.require()
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    width = (hq + 2 * hkv) * D
    if dout.stride(-1) != 1:
        dout = dout.contiguous()
    dqkv = torch.empty(B * S, width, dtype=qkv.dtype, device=qkv.device)
    acc = torch.empty(B * S, width, dtype=torch.float32, device=qkv.device)
    delta = torch.empty(B, hq, S, dtype=torch.float32, device=qkv.device)
    rc = lib.b200_flash_bwd(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), dout.data_ptr(), dout.stride(0),
                            lse.data_ptr(), delta.data_ptr(), acc.data_ptr(), dqkv.data_ptr(), B, S, hq, hkv, D, float(scale),
                            int(causal), _lib.err_word(qkv.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "flash_bwd")
    _count(3)
    return dqkv


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, B, S, hq, hkv, D, scale):
        out, lse = flash_fwd(qkv, B, S, hq, hkv, D, scale, True, True)
        ctx.save_for_backward(qkv, out, lse)
        ctx.dims = (B, S, hq, hkv, D, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        B, S, hq, hkv, D, scale = ctx.dims
        return flash_bwd(qkv, out, dout, lse, B, S, hq, hkv, D, scale, True), None, None, None, None, None, None


def flash_attention_packed(qkv, B, S, hq, hkv, D, scale: Optional[float] = None):
    if torch.is_grad_enabled() and qkv.requires_grad:
        return _FlashAttnFn.apply(qkv, B, S, hq, hkv, D, scale)
    out, _ = flash_fwd(qkv, B, S, hq, hkv, D, scale, True, False)
    return out
