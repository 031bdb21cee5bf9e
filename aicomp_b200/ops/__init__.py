"""Operator layer: hand-written sm_100a kernels with PyTorch reference fallbacks.

Dispatch rule, per call: CUDA + bf16 tensors run the kernels of the in-tree
library (and raise if it cannot be loaded); everything else (CPU tensors for
the gloo test paths, fp32 tensors) runs the plain PyTorch expression of the
same math, which is also the oracle the GPU tests compare against.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import check_errors, have_gpu_kernels  # noqa: F401

__all__ = [
    "gemm", "linear", "linear_kn", "rmsnorm", "layernorm", "rope_inplace", "apply_rope_qkv", "swiglu", "gelu_tanh", "cross_entropy",
    "embedding", "scaled_softmax", "check_errors", "have_gpu_kernels", "kernels_for", "launch_count", "reset_launch_count", "add_launches",
]

GEMM_OUT_F32 = 1
GEMM_ACCUMULATE = 2
GEMM_BIAS = 4

# Large GEMMs run on CTA pairs (two SMs per 256 x 256 tile); AICOMP_PAIR_GEMM=0 keeps every GEMM on the single-CTA kernel.
PAIR_GEMM = os.environ.get("AICOMP_PAIR_GEMM", "1") != "0"

_launches = 0


def _count(n: int = 1) -> None:
    global _launches
    _launches += n


def add_launches(n: int) -> None:
    """Account for kernels of this library that run inside a replayed CUDA graph."""
    _count(int(n))


def launch_count() -> int:
    """Number of kernels of this library launched since the last reset."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def kernels_for(*tensors: torch.Tensor) -> bool:
    """True when this call is served by the sm_100a kernels."""
    t0 = tensors[0]
    if not t0.is_cuda:
        return False
    if t0.dtype != torch.bfloat16:
        return False
    _lib.require()
    return True


def _rows(t: torch.Tensor) -> torch.Tensor:
    """View as 2D [rows, last] with unit inner stride (copy only if needed)."""
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(-1) != 1 or (t2.shape[0] > 1 and t2.stride(0) % 8 != 0) or t2.data_ptr() % 16 != 0:
        t2 = t2.contiguous()
    return t2


# ---------------------------------------------------------------------- GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: Optional[torch.Tensor] = None,
         out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False, bias: Optional[torch.Tensor] = None,
         alpha: float = 1.0, bn: int = 0, max_ctas: int = 0, ksplit: int = 1, pair: Optional[bool] = None) -> torch.Tensor:
    """``C[M,N] (+)= alpha * A @ B^T (+ bias)`` on tcgen05 tensor cores.

    ``pair``: run the CTA-pair kernel (``cta_group::2``, 256 x 256 tiles); default: whenever the problem is large
    enough for it (``PAIR_GEMM`` switches the default off).

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``), ``b`` is ``[N,K]`` (or
    ``[K,N]`` when ``b_mn``): the ``*_mn`` forms read a transposed operand in
    place, so dgrad and wgrad need no transposed copies.
    """
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"gemm: contraction mismatch {K} vs {Kb}")
    if out is not None:
        out_dtype = out.dtype
    if not kernels_for(a, b):
        af = (a.t() if a_mn else a).float()
        bf = (b.t() if b_mn else b).float()
        res = alpha * (af @ bf.t())
        if bias is not None:
            res = res + bias.float()
        if out is None:
            return res.to(out_dtype)
        if accumulate:
            out.add_(res.to(out.dtype))
        else:
            out.copy_(res.to(out.dtype))
        return out
    if a.stride(-1) != 1 or b.stride(-1) != 1:
        raise ValueError("gemm: operands need unit inner stride")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
        if accumulate:
            raise ValueError("gemm: accumulate needs out=")
    flags = (GEMM_OUT_F32 if out.dtype == torch.float32 else 0) | (GEMM_ACCUMULATE if accumulate else 0) | \
        (GEMM_BIAS if bias is not None else 0)
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("gemm: out must be bf16 or fp32")
    if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_contiguous()):
        bias = bias.to(torch.bfloat16).contiguous()
    lib = _lib.require()
    if pair is None:
        pair = PAIR_GEMM and bn == 0 and ksplit == 1
    if pair and ksplit == 1 and hasattr(lib, "b200_gemm2_bf16") and lib.b200_gemm2_supported(M, N, K):
        rc = lib.b200_gemm2_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(bias), M, N, K,
                                 a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn), flags, float(alpha),
                                 max_ctas, _lib.err_word(a.device).data_ptr(), _lib.stream_ptr())
    else:
        rc = lib.b200_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(bias), M, N, K,
                                a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn), flags, float(alpha),
                                bn, max_ctas, ksplit, _lib.err_word(a.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm")
    _count()
    return out


class _LinearFn(torch.autograd.Function):
    """y = x W^T + b with all three GEMMs on the tcgen05 kernel.

    When the weight carries a ``main_grad`` attribute (fp32 view into the
    optimizer's flat gradient arena) the weight gradient is accumulated there by
    the GEMM epilogue and no ``.grad`` tensor is produced.
    """

    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = _rows(x)
        # allocate with the final shape: a view made inside a Function may not be modified in place later (RoPE does)
        y = torch.empty(*x.shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)
        gemm(x2, w, bias=bias, out=y.view(-1, w.shape[0]))
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _rows(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(ctx.x_shape, dtype=dy.dtype, device=dy.device)
            gemm(dy2, w, b_mn=True, out=dx.view(-1, w.shape[1]))
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)
                ctx.w_ref.grad_accumulated = True
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


class _LinearKNFn(torch.autograd.Function):
    """y = x W + b for a weight stored ``[in, out]`` (HF ``Conv1D`` of the GPT-2 family): the GEMM reads W as an
    MN-major operand, so neither pass needs a transposed copy.  Same ``main_grad`` convention as :class:`_LinearFn`."""

    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = _rows(x)
        y = torch.empty(*x.shape[:-1], w.shape[1], dtype=x.dtype, device=x.device)
        gemm(x2, w, b_mn=True, bias=bias, out=y.view(-1, w.shape[1]))
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        ctx.w_ref = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _rows(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(ctx.x_shape, dtype=dy.dtype, device=dy.device)
            gemm(dy2, w, out=dx.view(-1, w.shape[0]))             # dx[M, in] = dy[M, out] . W[in, out]^T
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.w_ref, "main_grad", None)
            if mg is not None:
                gemm(x2, dy2, a_mn=True, b_mn=True, out=mg, accumulate=True)   # dW[in, out] = x^T dy
                ctx.w_ref.grad_accumulated = True
            else:
                dw = gemm(x2, dy2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear_kn(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w + bias`` with ``w`` stored ``[in_features, out_features]``."""
    if not kernels_for(x, w) or w.shape[0] % 8 or w.shape[1] % 8:
        y = x.reshape(-1, x.shape[-1]) @ w
        if bias is not None:
            y = y + bias
        return y.view(*x.shape[:-1], w.shape[1])
    return _LinearKNFn.apply(x, w, bias)


def _linear_small_m(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """Decode-sized GEMM (few rows): weight streaming is the bound, so K is split over enough CTAs to pull on all of
    HBM; partial products meet in an fp32 buffer through the reduce-add epilogue and are cast once."""
    x2 = _rows(x)
    M, K = x2.shape
    N = w.shape[0]
    tiles = ((M + 127) // 128) * ((N + 127) // 128)
    ks = max(1, min(16, (2 * 148) // max(tiles, 1), K // 512))
    if ks == 1:
        y = torch.empty(*x.shape[:-1], N, dtype=x.dtype, device=x.device)
        gemm(x2, w, bias=bias, out=y.view(-1, N), bn=128)
        return y
    acc = torch.zeros(M, N, dtype=torch.float32, device=x.device)
    gemm(x2, w, bias=bias, out=acc, accumulate=True, bn=128, ksplit=ks)
    return acc.to(x.dtype).view(*x.shape[:-1], N)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not kernels_for(x, w) or w.shape[0] % 8 or w.shape[1] % 8:   # e.g. a 10-class head: rows of C would not be 16-byte aligned
        return F.linear(x, w, bias)
    if not torch.is_grad_enabled() and x.numel() // x.shape[-1] <= 256:
        return _linear_small_m(x, w, bias)
    return _LinearFn.apply(x, w, bias)


# ---------------------------------------------------------------------- norms
_norm_scratch = {}


def _norm_scratch_for(device: torch.device, H: int) -> torch.Tensor:
    lib = _lib.require()
    n = 2 * lib.b200_norm_bwd_ctas() * H
    key = (device.index, )
    buf = _norm_scratch.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.empty(n, dtype=torch.float32, device=device)
        _norm_scratch[key] = buf
    return buf


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, b, eps, is_ln):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, H)
            if not r2.is_contiguous():
                r2 = r2.contiguous()
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        res_out = torch.empty(x.shape, dtype=x.dtype, device=x.device) if residual is not None else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device) if is_ln else None
        lib = _lib.require()
        rc = lib.b200_norm_fwd(x2.data_ptr(), _lib.ptr(r2), w.data_ptr(), _lib.ptr(b), y.data_ptr(), _lib.ptr(res_out),
                               rstd.data_ptr(), _lib.ptr(mean), rows, H, float(eps), int(is_ln), _lib.stream_ptr())
        _lib.check_rc(rc, "norm_fwd")
        _count()
        ctx.save_for_backward(res_out.view(-1, H) if res_out is not None else x2, w, rstd, mean)
        ctx.is_ln = is_ln
        ctx.has_res = residual is not None
        ctx.has_b = b is not None
        ctx.shape = x.shape
        ctx.w_ref, ctx.b_ref = w, b
        return y, res_out

    @staticmethod
    def backward(ctx, dy, dres):
        xin, w, rstd, mean = ctx.saved_tensors
        H = xin.shape[-1]
        rows = xin.shape[0]
        dy2 = dy.reshape(-1, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres2 = None
        if dres is not None:
            dres2 = dres.reshape(-1, H)
            if not dres2.is_contiguous():
                dres2 = dres2.contiguous()
        dx = torch.empty(ctx.shape, dtype=xin.dtype, device=xin.device)
        lib = _lib.require()
        scratch = _norm_scratch_for(xin.device, H)
        w_mg = getattr(ctx.w_ref, "main_grad", None)
        b_mg = getattr(ctx.b_ref, "main_grad", None) if ctx.has_b else None
        dw = db = None
        if w_mg is None:
            dw = torch.empty_like(w)
        if ctx.has_b and b_mg is None:
            db = torch.empty_like(w)
        rc = lib.b200_norm_bwd(dy2.data_ptr(), xin.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(mean), _lib.ptr(dres2),
                               dx.data_ptr(), scratch.data_ptr(), _lib.ptr(w_mg), _lib.ptr(dw), _lib.ptr(b_mg), _lib.ptr(db),
                               1 if w_mg is not None else 0, rows, H, int(ctx.is_ln), _lib.stream_ptr())
        _lib.check_rc(rc, "norm_bwd")
        _count(3 if ctx.is_ln and ctx.has_b else 2)
        if w_mg is not None:
            ctx.w_ref.grad_accumulated = True
        return dx, (dx if ctx.has_res else None), dw, db, None, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6, residual: Optional[torch.Tensor] = None
            ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``y = rmsnorm(x + residual) * w``; returns ``(y, x + residual)`` (second is None without residual)."""
    if not kernels_for(x) or x.shape[-1] % 8 or x.shape[-1] > 8192:
        r = x if residual is None else x + residual
        rf = r.float()
        y = (rf * torch.rsqrt(rf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w
        return y, (r if residual is not None else None)
    return _NormFn.apply(x, residual, w, None, eps, False)


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float = 1e-5,
              residual: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    if not kernels_for(x) or x.shape[-1] % 8 or x.shape[-1] > 8192:
        r = x if residual is None else x + residual
        y = F.layer_norm(r, (r.shape[-1],), w, b, eps)
        return y, (r if residual is not None else None)
    return _NormFn.apply(x, residual, w, b, eps, True)


# ---------------------------------------------------------------------- RoPE
_rope_cache = {}


def rope_tables(max_pos: int, dim: int, theta: float, device, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables ``[max_pos, dim/2]`` (HF default rope; optional llama3 frequency scaling); shared by all layers."""
    key = (max_pos, dim, float(theta), str(device), repr(sorted(scaling.items())) if scaling else None)
    hit = _rope_cache.get(key)
    if hit is None:
        hit = _rope_tables(max_pos, dim, theta, device, scaling)
        _rope_cache[key] = hit
    return hit


def _rope_tables(max_pos: int, dim: int, theta: float, device, scaling: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = scaling["factor"]
        lo, hi = scaling.get("low_freq_factor", 1.0), scaling.get("high_freq_factor", 4.0)
        old = scaling.get("original_max_position_embeddings", 8192)
        wavelen = 2 * math.pi / inv_freq
        smooth = ((old / wavelen) - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv_freq / factor, inv_freq)
        mid = (1 - smooth) * inv_freq / factor + smooth * inv_freq
        is_mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        inv_freq = torch.where(is_mid, mid, scaled)
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv_freq[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


def rope_inplace(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int,
                 head_dim: int, sign: float = 1.0) -> torch.Tensor:
    """Rotate the first ``n_rot_heads`` heads of every row of ``x [tokens, heads*head_dim]`` in place."""
    tokens = x.shape[0]
    if not kernels_for(x):
        xv = x[:, : n_rot_heads * head_dim].reshape(tokens, n_rot_heads, head_dim).float()
        c = cos[positions.long()][:, None, :]
        s = sin[positions.long()][:, None, :] * sign
        x1, x2 = xv[..., : head_dim // 2], xv[..., head_dim // 2:]
        out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
        x[:, : n_rot_heads * head_dim] = out.reshape(tokens, -1).to(x.dtype)
        return x
    if x.stride(-1) != 1:
        raise ValueError("rope: unit inner stride required")
    pos32 = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
    lib = _lib.require()
    rc = lib.b200_rope(x.data_ptr(), pos32.data_ptr(), cos.data_ptr(), sin.data_ptr(), tokens, n_rot_heads, head_dim,
                       x.stride(0), float(sign), _lib.stream_ptr())
    _lib.check_rc(rc, "rope")
    _count()
    return x


class _RopeQKVFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, positions, cos, sin, n_rot_heads, head_dim):
        ctx.mark_dirty(qkv)
        ctx.save_for_backward(positions, cos, sin)
        ctx.cfg = (n_rot_heads, head_dim)
        rope_inplace(qkv, positions, cos, sin, n_rot_heads, head_dim, 1.0)
        return qkv

    @staticmethod
    def backward(ctx, d):
        positions, cos, sin = ctx.saved_tensors
        d = d.clone(memory_format=torch.contiguous_format)  # the incoming gradient may be shared
        rope_inplace(d, positions, cos, sin, ctx.cfg[0], ctx.cfg[1], -1.0)
        return d, None, None, None, None, None


def apply_rope_qkv(qkv: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int,
                   head_dim: int) -> torch.Tensor:
    """Differentiable in-place RoPE on a packed ``[tokens, (Hq+2Hkv)*D]`` projection (q and k heads rotated)."""
    if not qkv.requires_grad:
        return rope_inplace(qkv, positions, cos, sin, n_rot_heads, head_dim)
    return _RopeQKVFn.apply(qkv, positions, cos, sin, n_rot_heads, head_dim)


# ---------------------------------------------------------------------- activations
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        I = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * I)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        out = torch.empty(*gu.shape[:-1], I, dtype=gu.dtype, device=gu.device)
        lib = _lib.require()
        _lib.check_rc(lib.b200_swiglu_fwd(g2.data_ptr(), out.data_ptr(), g2.shape[0], I, _lib.stream_ptr()), "swiglu_fwd")
        _count()
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        I = g2.shape[1] // 2
        d2 = dout.reshape(-1, I)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = torch.empty(ctx.shape, dtype=g2.dtype, device=g2.device)
        lib = _lib.require()
        _lib.check_rc(lib.b200_swiglu_bwd(g2.data_ptr(), d2.data_ptr(), dgu.data_ptr(), g2.shape[0], I, _lib.stream_ptr()), "swiglu_bwd")
        _count()
        return dgu


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for a packed ``[..., 2*I]`` (gate | up) tensor."""
    I = gate_up.shape[-1] // 2
    if not kernels_for(gate_up) or I % 8:
        return F.silu(gate_up[..., :I]) * gate_up[..., I:]
    return _SwiGLUFn.apply(gate_up)


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        lib = _lib.require()
        _lib.check_rc(lib.b200_gelu_fwd(xc.data_ptr(), y.data_ptr(), xc.numel(), _lib.stream_ptr()), "gelu_fwd")
        _count()
        ctx.save_for_backward(xc)
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        lib = _lib.require()
        _lib.check_rc(lib.b200_gelu_bwd(xc.data_ptr(), dyc.data_ptr(), dx.data_ptr(), xc.numel(), _lib.stream_ptr()), "gelu_bwd")
        _count()
        return dx


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    if not kernels_for(x) or x.numel() % 8:
        return F.gelu(x, approximate="tanh")
    return _GeluFn.apply(x)


# ---------------------------------------------------------------------- loss
class _CrossEntropyFn(torch.autograd.Function):
    """Mean token cross entropy; the logits buffer is overwritten by its own gradient in the forward."""

    @staticmethod
    def forward(ctx, logits, labels, ignore_index, unit_grad):
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V)
        if l2.stride(-1) != 1:
            l2 = l2.contiguous()
        lab = labels.reshape(-1)
        if lab.dtype != torch.int64:
            lab = lab.long()
        lab = lab.contiguous()
        rows = l2.shape[0]
        n_valid = (lab != ignore_index).sum().clamp_(min=1).float()
        loss_rows = torch.empty(rows, dtype=torch.float32, device=logits.device)
        need_grad = logits.requires_grad
        lib = _lib.require()
        inv = (1.0 / n_valid).reshape(1)
        rc = lib.b200_cross_entropy(l2.data_ptr(), lab.data_ptr(), loss_rows.data_ptr(), rows, V, l2.stride(0), int(ignore_index),
                                    1.0, inv.data_ptr(), int(need_grad), _lib.stream_ptr())
        _lib.check_rc(rc, "cross_entropy")
        _count()
        if need_grad:
            ctx.save_for_backward(l2)
            ctx.shape = logits.shape
            ctx.unit_grad = unit_grad
        return loss_rows.sum() * inv[0]

    @staticmethod
    def backward(ctx, dloss):
        (l2,) = ctx.saved_tensors
        if not ctx.unit_grad:  # the stored gradient is already d(mean loss)/d(logits); scale by the incoming gradient
            l2.mul_(dloss.to(l2.dtype))
        return l2.view(ctx.shape), None, None, None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100, unit_grad: bool = False) -> torch.Tensor:
    """Mean cross entropy over non-ignored tokens (fp32 math).  On the kernel path ``logits`` is consumed.

    ``unit_grad=True`` promises that ``backward`` starts from this loss with gradient 1 (what the pipeline
    schedules do), which saves a pass over the vocabulary-sized gradient."""
    V = logits.shape[-1]
    if not kernels_for(logits) or V % 8:
        return F.cross_entropy(logits.reshape(-1, V).float(), labels.reshape(-1).long(), ignore_index=ignore_index)
    return _CrossEntropyFn.apply(logits, labels, ignore_index, unit_grad)


# ---------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        idc = ids.reshape(-1).long().contiguous()
        H = table.shape[1]
        out = torch.empty(*ids.shape, H, dtype=table.dtype, device=table.device)
        lib = _lib.require()
        _lib.check_rc(lib.b200_embedding_fwd(idc.data_ptr(), table.data_ptr(), out.data_ptr(), idc.numel(), H, table.shape[0],
                                             _lib.stream_ptr()), "embedding_fwd")
        _count()
        ctx.save_for_backward(idc)
        ctx.t_ref = table
        return out

    @staticmethod
    def backward(ctx, dout):
        (idc,) = ctx.saved_tensors
        table = ctx.t_ref
        H = table.shape[1]
        d2 = dout.reshape(-1, H)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        mg = getattr(table, "main_grad", None)
        lib = _lib.require()
        if mg is not None:
            target = mg
        else:
            target = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        _lib.check_rc(lib.b200_embedding_bwd(idc.data_ptr(), d2.data_ptr(), target.data_ptr(), idc.numel(), H, table.shape[0],
                                             _lib.stream_ptr()), "embedding_bwd")
        _count()
        if mg is not None:
            table.grad_accumulated = True
            return None, None
        return None, target.to(table.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if not kernels_for(table) or table.shape[1] % 8:
        return F.embedding(ids, table)
    return _EmbeddingFn.apply(ids, table)


# ---------------------------------------------------------------------- softmax (parity with the reference's fused softmax kernels)
class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, scale, causal):
        xc = x.contiguous()
        b, h, sq, sk = xc.shape
        y = torch.empty_like(xc)
        mode = 2 if causal else (1 if mask is not None else 0)
        mb = 1
        mptr = None
        if mask is not None:
            m8 = mask.to(torch.uint8).contiguous()
            mb = m8.shape[0]
            mptr = m8.data_ptr()
        lib = _lib.require()
        rc = lib.b200_softmax_fwd(xc.data_ptr(), mptr, y.data_ptr(), b * h * sq, sq, sk, float(scale), mode, h, mb, _lib.stream_ptr())
        _lib.check_rc(rc, "softmax_fwd")
        _count()
        ctx.save_for_backward(y)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = torch.empty_like(y)
        sk = y.shape[-1]
        lib = _lib.require()
        rc = lib.b200_softmax_bwd(dyc.data_ptr(), y.data_ptr(), dx.data_ptr(), y.numel() // sk, sk, float(ctx.scale), _lib.stream_ptr())
        _lib.check_rc(rc, "softmax_bwd")
        _count()
        return dx, None, None, None


def scaled_softmax(x: torch.Tensor, scale: float = 1.0, mask: Optional[torch.Tensor] = None, causal: bool = False) -> torch.Tensor:
    """softmax(scale * x) over the last dim of ``[b, heads, sq, sk]``.

    ``mask`` (``[1 or b, 1, sq, sk]``, nonzero = masked) replaces scores by -10000 as the reference's
    ``scaled_masked_softmax``; ``causal`` zeroes the strictly-upper triangle as ``scaled_upper_triang_masked_softmax``.
    """
    if not kernels_for(x):
        s = x.float() * scale
        if mask is not None:
            s = s.masked_fill(mask.bool(), -10000.0)
        if causal:
            sq, sk = x.shape[-2:]
            keep = torch.ones(sq, sk, dtype=torch.bool, device=x.device).tril(sk - sq)
            s = s.masked_fill(~keep, float("-inf"))
        return torch.softmax(s, dim=-1).to(x.dtype)
    return _SoftmaxFn.apply(x, mask, scale, causal)
