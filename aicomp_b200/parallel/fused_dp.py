"""Fused data-parallel gradient all-reduce over peer memory.

The fp32 gradient arena of every data-parallel replica lives in a symmetric
buffer.  One call reduces a region in place with two kernels of this library
(no NCCL): each rank sums its 1/dp slice straight out of all peers' arenas over
NVLink, scales by 1/dp in the same pass, then pulls the other ranks' finished
slices.  Epoch flags written with system-scope release stores order the phases;
every wait is bounded and reports through the kernel status word.

Baseline it replaces: torch DDP's bucketed NCCL all-reduce followed by a divide
(opt_prime/opt_prime/opti_pri.py:852, schedule.py:851-864).
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import _lib
from .symm import FlagPad, SymmetricBuffer


class FusedGradAllReduce:
    SLOT = 0  # uses flag slots 0..2

    def __init__(self, group, dp_size: int, device: torch.device):
        if device.type != "cuda":
            raise RuntimeError("fused DP reduce needs CUDA")
        self.group, self.dp_size, self.device = group, dp_size, device
        self.flags = FlagPad(group, device)
        self.arena: SymmetricBuffer = None
        self.rank = self.flags.rank
        self._base = 0

    def alloc_arena(self, numel: int) -> torch.Tensor:
        """Collective: a zeroed fp32 tensor of ``numel`` elements in symmetric memory, to be used as the gradient arena."""
        self.arena = SymmetricBuffer(self.group, numel * 4, self.device)
        self._base = self.arena.ptrs[self.rank]
        return self.arena.view(torch.float32, numel)

    def supports(self, flat: torch.Tensor) -> bool:
        if self.arena is None or flat.dtype != torch.float32 or not flat.is_contiguous():
            return False
        off = flat.data_ptr() - self._base
        return 0 <= off and off + flat.numel() * 4 <= self.arena.nbytes and flat.numel() % 4 == 0 and off % 16 == 0

    def all_reduce_mean_(self, flat: torch.Tensor) -> None:
        lib = _lib.require()
        off = flat.data_ptr() - self._base
        epoch = self.flags.next_epoch(self.SLOT, span=3)
        rc = lib.b200_allreduce_mean_f32(self.arena.ptr_array(off), self.flags._ptrs, self.rank, self.dp_size, flat.numel(),
                                         self.SLOT, epoch, 0, _lib.err_word(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "allreduce_mean_f32")
        ops._count(6)

    def shard_bounds(self, numel: int):
        """Slice of an ``numel``-element region that this rank owns after :meth:`reduce_scatter_mean_`."""
        chunk = ((numel // 4 + self.dp_size - 1) // self.dp_size) * 4
        lo = min(self.rank * chunk, numel)
        return lo, min(lo + chunk, numel)

    def reduce_scatter_mean_(self, flat: torch.Tensor) -> None:
        """In place: this rank's slice of ``flat`` becomes the mean over the group (the other slices keep local values)."""
        lib = _lib.require()
        off = flat.data_ptr() - self._base
        epoch = self.flags.next_epoch(self.SLOT, span=3)
        rc = lib.b200_reduce_scatter_mean_f32(self.arena.ptr_array(off), self.flags._ptrs, self.rank, self.dp_size, flat.numel(),
                                              self.SLOT, epoch, 0, _lib.err_word(self.device).data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "reduce_scatter_mean_f32")
        ops._count(4)
