"""Data-parallel gradient reduction.

Gradients are reduced once per step, after the last micro-batch's backward (the
reference gates torch DDP the same way, opt_prime/opt_prime/schedule.py:851-864),
averaged over the data-parallel group.

``backend="nccl"``  flatten into ~64 MiB buckets, ``all_reduce`` on the group, scale,
                    copy back: the library baseline.
``backend="fused"`` one sm_100a kernel per bucket that reads every peer's bucket over
                    NVLink (symmetric memory), sums in fp32, scales by 1/dp and writes the
                    result in the gradient dtype (see ``parallel/fused_dp.py``); falls back
                    to ``nccl`` on CPU or when peer memory is unavailable.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..utils.log import get_logger

log = get_logger(__name__)

BUCKET_BYTES = 64 << 20


class GradReducer:
    def __init__(self, params: List[nn.Parameter], group, dp_size: int, backend: str = "fused", device=None):
        self.params = [p for p in params]
        self.group = group
        self.dp_size = dp_size
        self.device = device
        self.backend = backend
        self._fused = None
        self.bytes_reduced = 0
        if backend == "fused" and device is not None and device.type == "cuda":
            try:
                from .fused_dp import FusedGradAllReduce
                self._fused = FusedGradAllReduce(group, dp_size, device)
            except Exception as e:  # peer memory not available: keep the NCCL path
                log.warning("fused DP reduce unavailable (%r); using NCCL all-reduce", e)
                self._fused = None

    def broadcast_parameters(self, src: int) -> None:
        for p in self.params:
            dist.broadcast(p.data, src=src, group=self.group)

    def _grad_of(self, p: nn.Parameter) -> Optional[torch.Tensor]:
        if getattr(p, "grad_accumulated", False) and getattr(p, "main_grad", None) is not None:
            return p.main_grad
        return p.grad

    def reduce(self) -> None:
        pre = getattr(self, "pre_reduce", None)
        if pre is not None:
            pre()
        arena = getattr(self, "arena_grad", None)
        if arena is not None and getattr(self, "arena_mode", "all_reduce") == "reduce_scatter":
            # sharded optimizer: every rank needs the mean of its own slice only
            self.bytes_reduced += arena.numel() * arena.element_size()
            if self._fused is not None and self._fused.supports(arena):
                self._fused.reduce_scatter_mean_(arena)
            else:
                lo, hi = self.shard_bounds(arena.numel())
                chunk = ((arena.numel() // 4 + self.dp_size - 1) // self.dp_size) * 4
                if chunk * self.dp_size == arena.numel():
                    dist.reduce_scatter_tensor(arena[lo:hi], arena, group=self.group)
                    arena[lo:hi].div_(self.dp_size)
                else:
                    dist.all_reduce(arena, group=self.group)
                    arena.div_(self.dp_size)
            return
        if arena is not None:  # contiguous fp32 gradient arena (FusedAdamW): reduce it in place, bucket by bucket
            n = arena.numel()
            step = BUCKET_BYTES // arena.element_size()
            for off in range(0, n, step):
                self._reduce_flat(arena[off:min(off + step, n)])
            return
        grads = [g for g in (self._grad_of(p) for p in self.params if p.requires_grad) if g is not None]
        bucket: List[torch.Tensor] = []
        size = 0
        dtype = None
        for g in grads:
            nbytes = g.numel() * g.element_size()
            if bucket and (size + nbytes > BUCKET_BYTES or g.dtype != dtype):
                self._reduce_bucket(bucket)
                bucket, size = [], 0
            bucket.append(g)
            dtype = g.dtype
            size += nbytes
        if bucket:
            self._reduce_bucket(bucket)

    def shard_bounds(self, numel: int):
        """Slice [lo, hi) of a flat ``numel``-element arena owned by this rank of the data-parallel group."""
        rank = dist.get_rank(self.group)
        chunk = ((numel // 4 + self.dp_size - 1) // self.dp_size) * 4
        lo = min(rank * chunk, numel)
        return lo, min(lo + chunk, numel)

    def _reduce_flat(self, flat: torch.Tensor) -> None:
        self.bytes_reduced += flat.numel() * flat.element_size()
        if self._fused is not None and self._fused.supports(flat):
            self._fused.all_reduce_mean_(flat)
            return
        dist.all_reduce(flat, group=self.group)
        flat.div_(self.dp_size)

    def _reduce_bucket(self, bucket: List[torch.Tensor]) -> None:
        if len(bucket) == 1 and bucket[0].is_contiguous():
            self._reduce_flat(bucket[0].view(-1))
            return
        flat = torch.cat([g.reshape(-1) for g in bucket])
        self._reduce_flat(flat)
        off = 0
        for g in bucket:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g))
            off += n
