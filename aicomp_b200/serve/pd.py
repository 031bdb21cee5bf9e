"""Prefill/decode disaggregation: KV-cache page transfer between GPU groups.

Prefill GPUs compute a prompt's KV pages into their own page pool; the pages
are then *pushed* into the decode GPU's pool by a kernel of this library that
stores over NVLink (``b200_kv_push``) and raises the request's ready word only
after the page data is visible system-wide.  The decode side polls that word on
the host (or waits for it on its stream) before it schedules the request, so
hand-off ordering needs no host round trip between the two GPUs.

The reference has no KV transfer (its cache is a dense per-process tensor,
opt_prime/opt_prime/kv_cache.py:19-254); the baseline for this path is a
``cudaMemcpyPeerAsync`` / NCCL send per page.
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from ..ops import _lib
from .. import ops
from ..parallel.symm import SymmetricBuffer


class KVPagePusher:
    """Symmetric KV page pools ``[layers, 2, pool_pages, page_bytes]`` plus per-request ready words."""

    def __init__(self, group, device: torch.device, layers: int, pool_pages: int, page_bytes: int, request_slots: int = 4096):
        self.layers, self.pool_pages, self.page_bytes = layers, pool_pages, page_bytes
        self.device = device
        self.pool = SymmetricBuffer(group, layers * 2 * pool_pages * page_bytes, device)
        self.ready = SymmetricBuffer(group, request_slots * 4, device)
        self.rank, self.world = self.pool.rank, self.pool.world
        self.local_pool = self.pool.local[: layers * 2 * pool_pages * page_bytes].view(layers, 2, pool_pages, page_bytes)
        self.ready_words = self.ready.view(torch.int32, request_slots)
        self._counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.bytes_pushed = 0

    def push(self, dst_rank: int, src_pages: torch.Tensor, dst_pages: torch.Tensor, request_slot: Optional[int] = None,
             ready_value: int = 1) -> None:
        """Copy pages ``src_pages`` of the local pool to ``dst_pages`` of rank ``dst_rank``'s pool (all layers, K and V)."""
        lib = _lib.require()
        n = int(src_pages.numel())
        if n != int(dst_pages.numel()):
            raise ValueError("src_pages and dst_pages differ in length")
        sp = src_pages.to(device=self.device, dtype=torch.int32).contiguous()
        dp = dst_pages.to(device=self.device, dtype=torch.int32).contiguous()
        ready_ptr = None if request_slot is None else self.ready.ptrs[dst_rank] + 4 * request_slot
        rc = lib.b200_kv_push(self.pool.ptrs[self.rank], self.pool.ptrs[dst_rank], sp.data_ptr(), dp.data_ptr(), n, self.layers,
                              self.pool_pages, self.pool_pages, self.page_bytes, ready_ptr, ready_value,
                              self._counter.data_ptr(), _lib.stream_ptr())
        _lib.check_rc(rc, "kv_push")
        ops._count()
        self.bytes_pushed += n * self.layers * 2 * self.page_bytes
        self._keep = (sp, dp)

    def wait_ready(self, request_slot: int, ready_value: int, timeout_s: float = 10.0) -> bool:
        """Host-side poll of this rank's ready word; returns False when the time limit runs out."""
        t0 = time.time()
        while time.time() - t0 < timeout_s:
            if int(self.ready_words[request_slot].item()) == ready_value:
                return True
            time.sleep(0.0005)
        return False

    def clear_ready(self, request_slot: int) -> None:
        self.ready_words[request_slot] = 0
