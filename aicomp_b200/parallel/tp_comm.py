"""Differentiable tensor-/sequence-parallel communication primitives.

``nccl`` backend: plain ``torch.distributed`` collectives around the GEMMs (the
reference behaviour: DTensor redistributions that issue NCCL all-reduces,
opt_prime/opt_prime/opti_pri.py:887-1008).  ``fused`` backend: the all-gather is
pulled tile-by-tile from peer memory inside the GEMM's producer and the
reduce-scatter is pushed from the GEMM's epilogue (see ``parallel/fused_tp.py``).
Conventions: activations are ``[B, S, H]``; sequence parallelism shards dim 1.
"""
from __future__ import annotations


import torch
import torch.distributed as dist

from .. import ops


def _all_reduce(t: torch.Tensor, group) -> torch.Tensor:
    if group is not None:
        dist.all_reduce(t, group=group)
    return t


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel GEMM)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g.contiguous(), ctx.group), None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel GEMM)."""

    @staticmethod
    def forward(ctx, x, group):
        return _all_reduce(x.contiguous(), group)

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_tp(x, group):
    return _CopyToTP.apply(x, group)


def reduce_from_tp(x, group):
    return _ReduceFromTP.apply(x, group)


def _gather_seq(x: torch.Tensor, group, size: int) -> torch.Tensor:
    """[B, S/tp, H] on every rank -> [B, S, H]."""
    B, S_loc, H = x.shape
    xc = x.contiguous()
    if B == 1:
        out = torch.empty(1, S_loc * size, H, dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out.view(size * S_loc, H), xc.view(S_loc, H), group=group)
        return out
    buf = torch.empty(size * B, S_loc, H, dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(buf, xc, group=group)
    return buf.view(size, B, S_loc, H).permute(1, 0, 2, 3).reshape(B, size * S_loc, H)


def _reduce_scatter_seq(x: torch.Tensor, group, size: int) -> torch.Tensor:
    """[B, S, H] partial sums on every rank -> [B, S/tp, H] reduced shard."""
    B, S, H = x.shape
    S_loc = S // size
    if not x.is_cuda:  # gloo has no reduce-scatter: all-reduce and keep this rank's slice
        full = x.contiguous().clone()
        dist.all_reduce(full, group=group)
        r = dist.get_rank(group)
        return full[:, r * S_loc:(r + 1) * S_loc].contiguous()
    if B == 1:
        out = torch.empty(1, S_loc, H, dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out.view(S_loc, H), x.contiguous().view(S, H), group=group)
        return out
    xin = x.view(B, size, S_loc, H).permute(1, 0, 2, 3).contiguous().view(size * B, S_loc, H)
    out = torch.empty(B, S_loc, H, dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, xin, group=group)
    return out


class _GatherSeq(torch.autograd.Function):
    """All-gather along the sequence forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, group, size):
        ctx.group, ctx.size = group, size
        return _gather_seq(x, group, size)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_seq(g, ctx.group, ctx.size), None, None


class _ReduceScatterSeq(torch.autograd.Function):
    """Reduce-scatter along the sequence forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, group, size):
        ctx.group, ctx.size = group, size
        return _reduce_scatter_seq(x, group, size)

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g, ctx.group, ctx.size), None, None


class _ScatterToSP(torch.autograd.Function):
    """Keep this rank's sequence shard of a replicated tensor; backward all-gathers the shard gradients."""

    @staticmethod
    def forward(ctx, x, group, rank, size):
        ctx.group, ctx.size = group, size
        S_loc = x.shape[1] // size
        return x[:, rank * S_loc:(rank + 1) * S_loc].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g, ctx.group, ctx.size), None, None, None


class _GatherFromSP(torch.autograd.Function):
    """All-gather the sequence shards into a replicated tensor; backward keeps this rank's slice."""

    @staticmethod
    def forward(ctx, x, group, rank, size):
        ctx.rank, ctx.size = rank, size
        return _gather_seq(x, group, size)

    @staticmethod
    def backward(ctx, g):
        S_loc = g.shape[1] // ctx.size
        return g[:, ctx.rank * S_loc:(ctx.rank + 1) * S_loc].contiguous(), None, None, None


def gather_seq(x, group, size):
    return _GatherSeq.apply(x, group, size)


def reduce_scatter_seq(x, group, size):
    return _ReduceScatterSeq.apply(x, group, size)


def scatter_to_sp(x, group, rank, size):
    if x.shape[1] % size:
        raise ValueError(f"sequence length {x.shape[1]} is not divisible by tp_size {size}")
    return _ScatterToSP.apply(x, group, rank, size)


def gather_from_sp(x, group, rank, size):
    return _GatherFromSP.apply(x, group, rank, size)


def allgather_linear(x: torch.Tensor, w: torch.Tensor, group, size: int, backend: str = "nccl") -> torch.Tensor:
    """``all_gather_seq(x) @ w^T`` for a column-parallel weight shard ``w [N/tp, K]``."""
    if backend == "fused":
        from . import fused_tp
        if fused_tp.usable_ag(x, w, group):
            return fused_tp.allgather_gemm(x, w, group, size)
    return ops.linear(_GatherSeq.apply(x, group, size), w)


def linear_reducescatter(x: torch.Tensor, w: torch.Tensor, group, size: int, backend: str = "nccl") -> torch.Tensor:
    """``reduce_scatter_seq(x @ w^T)`` for a row-parallel weight shard ``w [N, K/tp]``."""
    if backend == "fused":
        from . import fused_tp
        if fused_tp.usable_rs(x, w, group):
            return fused_tp.gemm_reducescatter(x, w, group, size)
    return _ReduceScatterSeq.apply(ops.linear(x, w), group, size)
