"""Fused tensor-parallel GEMM + collective kernels over peer memory (sequence-parallel layout).

``allgather_gemm``      Y[T, N/tp] = all_gather_rows(X)[T, K] @ W^T.  Every rank publishes its row shard of X in a
                        peer-mapped buffer; the tcgen05 GEMM kernel of each rank reads the other shards' tiles
                        directly from the owners' HBM with (non-multicast) TMA loads, starting with its own rows
                        while the owners' ready flags are still in flight - no gathered copy of X is ever made.
``gemm_reducescatter``  Y[T/tp, N] = reduce_scatter_rows(X[T, K/tp] @ W^T).  The GEMM epilogue stores each
                        output tile with TMA straight into the staging slot of the rank that owns those rows
                        (remote rows first, so NVLink traffic overlaps the remaining tiles); after a flag
                        barrier every rank sums the tp partial slots it received.

The baseline they replace is NCCL all-gather / reduce-scatter around a separate GEMM (the reference: DTensor
column/row-wise redistributions, opt_prime/opt_prime/opti_pri.py:893-1008).  Both functions are differentiable:
the input-gradient of one is the other, and the weight gradients gather their second operand with NCCL.
"""
from __future__ import annotations

import ctypes
from typing import Dict

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib
from .symm import FlagPad, SymmetricBuffer

P = ctypes.c_void_p
_lib.OPTIONAL_PROTOS.update({
    "b200_gemm_bf16_parts": [ctypes.POINTER(P), _lib.I, _lib.I, P, ctypes.POINTER(P), _lib.I, _lib.I, P, _lib.I, _lib.I, _lib.I, _lib.L,
                             _lib.L, _lib.L, _lib.I, _lib.I, _lib.I, _lib.F, _lib.I, _lib.I, P, ctypes.c_uint, P, P],
    "b200_sum_parts_bf16": [P, _lib.I, _lib.L, P, _lib.L, P],
    "b200_ag_gemm_bf16": [P, ctypes.POINTER(P), ctypes.POINTER(P), _lib.I, _lib.I, _lib.I, ctypes.c_uint, P, P, P, _lib.I, _lib.I, _lib.I,
                          _lib.L, _lib.L, _lib.I, P, P],
    "b200_ag_gemm_bf16_dev": [P, ctypes.POINTER(P), ctypes.POINTER(P), _lib.I, _lib.I, _lib.I, P, P, P, P, _lib.I, _lib.I, _lib.I,
                              _lib.L, _lib.L, _lib.I, P, P],
    "b200_epoch_bump": [P, P],
    "b200_signal_dev": [ctypes.POINTER(P), _lib.I, _lib.I, _lib.I, P, P],
    "b200_wait_dev": [P, _lib.I, _lib.I, P, P, P],
})
_lib.rebind()

SLOT_AG_READY, SLOT_AG_DONE, SLOT_RS_READY, SLOT_RS_DONE = 8, 10, 12, 14
_contexts: Dict[int, "TPContext"] = {}


class TPContext:
    """Per tensor-parallel group: flag pad plus double-buffered symmetric staging for shards and partial results."""

    def __init__(self, group, device: torch.device):
        self.group, self.device = group, device
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.flags = FlagPad(group, device)
        self.ag_bufs = [None, None]
        self.rs_bufs = [None, None]
        self.ag_calls = 0
        self.rs_calls = 0
        self.counter = None
        # One epoch per flag slot, in DEVICE memory: it is bumped, published and waited for by kernels in stream
        # order, so a captured sequence of these launches replays correctly (no host-side counter is baked in).
        self.epochs = torch.zeros(64, dtype=torch.int32, device=device)

    def _eptr(self, slot: int) -> int:
        return self.epochs.data_ptr() + 4 * slot

    def bump(self, slot: int) -> None:
        _lib.check_rc(_lib.require().b200_epoch_bump(self._eptr(slot), _lib.stream_ptr()), "epoch_bump")

    def signal(self, slot: int, epoch_slot: int) -> None:
        """Publish the current epoch of ``epoch_slot`` in flag ``slot`` of every peer."""
        _lib.check_rc(_lib.require().b200_signal_dev(self.flags._ptrs, self.rank, self.size, slot, self._eptr(epoch_slot),
                                                     _lib.stream_ptr()), "signal_dev")

    def wait(self, slot: int, epoch_slot: int) -> None:
        """Wait (bounded) until every peer's flag ``slot`` has reached the current epoch of ``epoch_slot``."""
        _lib.check_rc(_lib.require().b200_wait_dev(self.flags.buf.ptrs[self.rank], self.size, slot, self._eptr(epoch_slot),
                                                   _lib.err_word(self.device).data_ptr(), _lib.stream_ptr()), "wait_dev")

    def _buf(self, bufs, i: int, nbytes: int) -> SymmetricBuffer:
        b = bufs[i]
        if b is None or b.nbytes < nbytes:
            # growing a buffer is collective; every rank reaches this with the same sizes (SPMD)
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            if b is not None:
                b.close()
            b = SymmetricBuffer(self.group, nbytes, self.device)
            bufs[i] = b
        return b


def context(group, device: torch.device) -> TPContext:
    key = id(group)
    c = _contexts.get(key)
    if c is None:
        c = TPContext(group, device)
        _contexts[key] = c
    return c


def _base_ok(x: torch.Tensor, w: torch.Tensor, group) -> bool:
    if group is None or not x.is_cuda or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    lib = _lib.require()
    if not hasattr(lib, "b200_gemm_bf16_parts"):
        return False
    if x.dim() == 3 and x.shape[0] != 1:
        return False  # the sequence shards of a batch > 1 are not contiguous row blocks
    return x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0


def usable_ag(x: torch.Tensor, w: torch.Tensor, group) -> bool:
    """``x`` holds this rank's sequence shard: its row count must be a multiple of the 128-row tile."""
    return _base_ok(x, w, group) and (x.numel() // x.shape[-1]) % 128 == 0


def usable_rs(x: torch.Tensor, w: torch.Tensor, group) -> bool:
    """``x`` holds all rows: every rank's share of them must be a multiple of the 128-row tile."""
    if not _base_ok(x, w, group):
        return False
    rows = x.numel() // x.shape[-1]
    size = dist.get_world_size(group)
    return rows % size == 0 and (rows // size) % 128 == 0


def _ag_gemm_raw(x_local: torch.Tensor, w: torch.Tensor, group, b_mn: bool = False) -> torch.Tensor:
    """x_local [T/tp, K] (this rank's rows), w [N, K] (or [K, N] when b_mn) -> [T, N]; one kernel pushes, waits and multiplies."""
    lib = _lib.require()
    ctx = context(group, x_local.device)
    tp, rank = ctx.size, ctx.rank
    Tl, K = x_local.shape
    N = w.shape[1] if b_mn else w.shape[0]
    if Tl % 128 or K % 8 or N % 8:
        raise ValueError("fused all-gather GEMM needs T/tp % 128 == 0")
    if not x_local.is_contiguous():
        x_local = x_local.contiguous()
    i = ctx.ag_calls & 1
    ctx.ag_calls += 1
    buf = ctx._buf(ctx.ag_bufs, i, tp * Tl * K * 2)  # gather buffer: one slot per rank
    # every peer has finished reading (its GEMM of two calls ago) what we are about to overwrite in its buffer: its
    # "done" flag carries the epoch this buffer had then (all flags start at the initial epoch 0)
    ctx.wait(SLOT_AG_DONE + i, SLOT_AG_READY + i)
    ctx.bump(SLOT_AG_READY + i)
    if ctx.counter is None:
        ctx.counter = torch.zeros(4, dtype=torch.int32, device=x_local.device)
    out = torch.empty(Tl * tp, N, dtype=x_local.dtype, device=x_local.device)
    rc = lib.b200_ag_gemm_bf16_dev(x_local.data_ptr(), buf.ptr_array(), ctx.flags._ptrs, rank, tp, SLOT_AG_READY + i,
                                   ctx._eptr(SLOT_AG_READY + i), ctx.counter.data_ptr(), w.data_ptr(), out.data_ptr(), Tl * tp, N, K,
                                   w.stride(0), out.stride(0), int(b_mn), _lib.err_word(x_local.device).data_ptr(),
                                   _lib.stream_ptr())
    _lib.check_rc(rc, "ag_gemm")
    ctx.signal(SLOT_AG_DONE + i, SLOT_AG_READY + i)
    ops._count(4)
    return out


def _gemm_rs_raw(x: torch.Tensor, w: torch.Tensor, group, b_mn: bool = False) -> torch.Tensor:
    """x [T, K/tp], w [N, K/tp] (or [K/tp, N] when b_mn) -> this rank's rows [T/tp, N] of the summed product."""
    lib = _lib.require()
    ctx = context(group, x.device)
    tp, rank = ctx.size, ctx.rank
    T, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    Tl = T // tp
    if T % tp or Tl % 128 or K % 8 or N % 8:
        raise ValueError("fused GEMM reduce-scatter needs T/tp % 128 == 0")
    j = ctx.rs_calls & 1
    ctx.rs_calls += 1
    slot_elems = Tl * N
    buf = ctx._buf(ctx.rs_bufs, j, tp * slot_elems * 2)
    # owners have summed (and so finished reading) what we stored there two calls ago
    ctx.wait(SLOT_RS_DONE + j, SLOT_RS_READY + j)
    ctx.bump(SLOT_RS_READY + j)
    a_parts = (P * 1)(x.data_ptr())
    c_parts = (P * tp)(*[buf.ptrs[o] + rank * slot_elems * 2 for o in range(tp)])
    rot = ((rank + 1) % tp) * (Tl // 128)
    rc = lib.b200_gemm_bf16_parts(a_parts, 1, 0, w.data_ptr(), c_parts, tp, Tl, None, T, N, K, x.stride(0), w.stride(0), N,
                                  0, int(b_mn), 0, 1.0, 0, rot, None, 0, _lib.err_word(x.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_rs")
    ctx.signal(SLOT_RS_READY + j, SLOT_RS_READY + j)
    ctx.wait(SLOT_RS_READY + j, SLOT_RS_READY + j)
    out = torch.empty(Tl, N, dtype=x.dtype, device=x.device)
    rc = lib.b200_sum_parts_bf16(buf.ptrs[rank], tp, slot_elems, out.data_ptr(), slot_elems, _lib.stream_ptr())
    _lib.check_rc(rc, "sum_parts")
    ctx.signal(SLOT_RS_DONE + j, SLOT_RS_READY + j)
    ops._count(7)
    return out


def _nccl_gather_rows(x_local: torch.Tensor, group, tp: int) -> torch.Tensor:
    out = torch.empty(x_local.shape[0] * tp, x_local.shape[1], dtype=x_local.dtype, device=x_local.device)
    dist.all_gather_into_tensor(out, x_local.contiguous(), group=group)
    return out


class _AGGemmFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group, size):
        x2 = x.reshape(-1, x.shape[-1])
        y = _ag_gemm_raw(x2.contiguous(), w, group)
        ctx.save_for_backward(x2, w)
        ctx.group, ctx.size, ctx.w_ref, ctx.x_shape = group, size, w, x.shape
        return y  # 2-D; reshaped by the caller (a view made inside a Function could not be modified in place later)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = _gemm_rs_raw(dy2, w, ctx.group, b_mn=True).view(ctx.x_shape)
        x_full = _nccl_gather_rows(x2, ctx.group, ctx.size)
        dw = None
        mg = getattr(ctx.w_ref, "main_grad", None)
        if mg is not None:
            ops.gemm(dy2, x_full, a_mn=True, b_mn=True, out=mg, accumulate=True)
            ctx.w_ref.grad_accumulated = True
        else:
            dw = ops.gemm(dy2, x_full, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw, None, None


class _GemmRSFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, group, size):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = _gemm_rs_raw(x2, w, group)
        ctx.save_for_backward(x2, w)
        ctx.group, ctx.size, ctx.w_ref, ctx.x_shape = group, size, w, x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = _ag_gemm_raw(dy2, w, ctx.group, b_mn=True).view(ctx.x_shape)
        dy_full = _nccl_gather_rows(dy2, ctx.group, ctx.size)
        dw = None
        mg = getattr(ctx.w_ref, "main_grad", None)
        if mg is not None:
            ops.gemm(dy_full, x2, a_mn=True, b_mn=True, out=mg, accumulate=True)
            ctx.w_ref.grad_accumulated = True
        else:
            dw = ops.gemm(dy_full, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw, None, None


def allgather_gemm(x: torch.Tensor, w: torch.Tensor, group, size: int) -> torch.Tensor:
    return _AGGemmFn.apply(x, w, group, size).view(1, -1, w.shape[0])


def gemm_reducescatter(x: torch.Tensor, w: torch.Tensor, group, size: int) -> torch.Tensor:
    return _GemmRSFn.apply(x, w, group, size).view(1, -1, w.shape[0])
