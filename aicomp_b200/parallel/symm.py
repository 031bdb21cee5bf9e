"""Symmetric (peer-mapped) device memory for a process group on one NVSwitch domain.

Each rank allocates a buffer with ``cudaMalloc``, exports it with CUDA IPC, and
opens every peer's export; kernels then take the table of per-rank base
pointers and read or write a peer's HBM directly over NVLink.  A small flag pad
per buffer carries the epochs that the signal/wait kernels exchange.

The reference has no custom transport (NCCL only); this layer is what the fused
compute+collective kernels of this framework stand on.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib

P = ctypes.c_void_p
_lib.OPTIONAL_PROTOS.update({
    "b200_symm_alloc": [ctypes.c_longlong, ctypes.POINTER(P), ctypes.c_char_p],
    "b200_symm_open": [ctypes.c_char_p, ctypes.POINTER(P)],
    "b200_symm_close": [P],
    "b200_symm_free": [P],
    "b200_signal": [ctypes.POINTER(P), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint, P],
    "b200_wait": [P, ctypes.c_int, ctypes.c_int, ctypes.c_uint, P, P],
    "b200_allreduce_mean_f32": [ctypes.POINTER(P), ctypes.POINTER(P), ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                                ctypes.c_uint, ctypes.c_int, P, P],
    "b200_reduce_scatter_mean_f32": [ctypes.POINTER(P), ctypes.POINTER(P), ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                                     ctypes.c_uint, ctypes.c_int, P, P],
    "b200_peer_pull": [P, P, ctypes.c_longlong, ctypes.c_int, P],
    "b200_stream_store_flag": [P, ctypes.c_uint, P],
    "b200_stream_wait_flag_geq": [P, ctypes.c_uint, P],
    "b200_copy_async": [P, P, ctypes.c_longlong, P],
    "b200_kv_push": [P, P, P, P, ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int, P, ctypes.c_uint,
                     P, P],
})

_lib.rebind()

FLAG_SLOTS = 64
MAX_PEERS = 8


class _RawCudaArray:
    """Minimal ``__cuda_array_interface__`` carrier so torch can view memory it did not allocate."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


def _tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.as_tensor(_RawCudaArray(ptr, nbytes), device=device)


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``group``, mapped into every rank.

    ``local`` is this rank's memory as a uint8 tensor; ``ptrs[r]`` is rank r's base address as seen
    from this process.  Construction is collective over ``group``.
    """

    def __init__(self, group, nbytes: int, device: torch.device):
        lib = _lib.require()
        if not hasattr(lib, "b200_symm_alloc"):
            raise RuntimeError("kernel library was built without symmetric-memory support")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > MAX_PEERS:
            raise ValueError(f"symmetric buffers support up to {MAX_PEERS} peers")
        self.device = device
        self.nbytes = int((nbytes + 255) // 256 * 256)
        ptr = P()
        handle = ctypes.create_string_buffer(64)
        _lib.check_rc(lib.b200_symm_alloc(self.nbytes, ctypes.byref(ptr), handle), "symm_alloc")
        self._own = ptr.value
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self._own)
                continue
            q = P()
            _lib.check_rc(lib.b200_symm_open(h, ctypes.byref(q)), "symm_open")
            self.ptrs.append(q.value)
            self._opened.append(q.value)
        self.local = _tensor_from_ptr(self._own, self.nbytes, device)
        self._keep = (handle,)

    def ptr_array(self, offset: int = 0):
        arr = (P * self.world)(*[p + offset for p in self.ptrs])
        return arr

    def view(self, dtype: torch.dtype, numel: Optional[int] = None, offset_bytes: int = 0) -> torch.Tensor:
        t = self.local[offset_bytes:].view(dtype)
        return t if numel is None else t[:numel]

    def close(self) -> None:
        lib = _lib.load()
        if lib is None:
            return
        for p in self._opened:
            lib.b200_symm_close(p)
        self._opened = []
        if self._own:
            self.local = None
            lib.b200_symm_free(self._own)
            self._own = 0


class FlagPad:
    """Symmetric array of ``FLAG_SLOTS x MAX_PEERS`` 32-bit epochs plus a per-slot host-side epoch counter."""

    def __init__(self, group, device: torch.device):
        self.buf = SymmetricBuffer(group, FLAG_SLOTS * MAX_PEERS * 4, device)
        self.epochs = [0] * FLAG_SLOTS
        self.rank, self.world = self.buf.rank, self.buf.world
        self._ptrs = self.buf.ptr_array()

    def next_epoch(self, slot: int, span: int = 1) -> int:
        e = self.epochs[slot] + 1
        for s in range(slot, slot + span):
            self.epochs[s] = e
        return e

    def signal(self, slot: int, epoch: int) -> None:
        lib = _lib.require()
        _lib.check_rc(lib.b200_signal(self._ptrs, self.rank, self.world, slot, epoch, _lib.stream_ptr()), "signal")

    def wait(self, slot: int, epoch: int) -> None:
        lib = _lib.require()
        _lib.check_rc(lib.b200_wait(self.buf.ptrs[self.rank], self.world, slot, epoch, _lib.err_word(self.buf.device).data_ptr(),
                                    _lib.stream_ptr()), "wait")

    def barrier(self, slot: int) -> None:
        """Device-side barrier of the group on the current stream (no host synchronisation)."""
        e = self.next_epoch(slot)
        self.signal(slot, e)
        self.wait(slot, e)
