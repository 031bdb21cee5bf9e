"""Pipeline point-to-point transport over peer-mapped memory (one NVSwitch domain), without NCCL kernels.

A receive posted early through NCCL is a kernel that sits on the GPU until the matching send arrives.  The GEMM kernels
of this framework are persistent, one CTA per SM with almost all of its shared memory: an SM that holds a waiting
NCCL CTA cannot take its GEMM CTA, which then runs after the others have finished - under 1F1B, where a receive is
nearly always pending, a stage's kernels ran about 17 % slower than the same kernels on a single GPU.

:class:`PeerChannel` keeps the interface of :class:`~aicomp_b200.parallel.comm.Channel` and moves the payload with
primitives that occupy no SM while they wait:

* the receiver owns a ring of ``RING`` slots in its own memory, mapped into the sender through CUDA IPC;
* ``send`` waits (stream memory operation on a flag in the sender's memory) until the slot's previous message was
  consumed, copies the tensors into the slot with the copy engines, and stores the message number into the slot's
  ``full`` flag in the receiver's memory - all on the current stream, nothing blocks the host;
* ``wait_recv`` makes the current stream wait for the ``full`` flag (stream memory operation), copies the slot into
  ordinary tensors and stores the message number into the slot's ``free`` flag in the sender's memory.

The header (tree structure, shapes, dtypes) still travels through the process group, once per step, as in ``Channel``.
The reference moves every tensor with NCCL ``isend``/``irecv`` (opt_prime/opt_prime/comm.py:60-230).
"""
from __future__ import annotations

from typing import Any, List

import torch
import torch.distributed as dist

from ..ops import _lib
from .comm import Channel, Comm, _decode, _encode, _same_signature
from .symm import SymmetricBuffer

# the stream-flag and copy entry points are declared with the other symmetric-memory prototypes (parallel/symm.py)

RING = 4          # slots per channel; flow control makes any value >= 1 correct
_ALIGN = 256
_FLAG_BYTES = 256  # RING 'full' flags then RING 'free' flags, 4 bytes each, padded


def peer_transport_available(device: torch.device) -> bool:
    lib = _lib.load()
    return device.type == "cuda" and lib is not None and hasattr(lib, "b200_stream_wait_flag_geq")


class PeerChannel(Channel):
    """One direction of pipeline traffic between two ranks of one node, through a ring in the receiver's memory."""

    def __init__(self, comm: Comm, src: int, dst: int, tag: str, group):
        super().__init__(comm, src, dst, tag, group)
        self.buf: SymmetricBuffer | None = None
        self.slot_bytes = 0
        self.seq = 0            # messages sent / received so far on this channel
        self._offsets: List[int] = []
        self._expected = 0      # receives posted and not yet waited for
        self._peer = 1 - dist.get_rank(group)
        self._me = dist.get_rank(group)

    # -- layout --------------------------------------------------------------
    def _layout(self, metas) -> int:
        self._offsets, off = [], 0
        for dtype, shape, _ in metas:
            n = 1
            for d in shape:
                n *= d
            self._offsets.append(off)
            off += (n * torch.empty((), dtype=dtype).element_size() + _ALIGN - 1) // _ALIGN * _ALIGN
        return max(off, _ALIGN)

    def _ensure_ring(self, metas) -> None:
        """Collective over the pair: (re)allocate the ring when the payload no longer fits a slot."""
        need = self._layout(metas)
        if self.buf is not None and need <= self.slot_bytes:
            return
        torch.cuda.synchronize(self.comm.device)
        if self.buf is not None:
            dist.barrier(group=self.group)  # both sides are past every message of the old ring
            self.buf.close()
        self.slot_bytes = need
        self.buf = SymmetricBuffer(self.group, _FLAG_BYTES + RING * need, self.comm.device)
        self.seq = 0

    def _flag(self, owner: int, kind: int, slot: int) -> int:
        return self.buf.ptrs[owner] + (kind * RING + slot) * 4

    def _slot(self, owner: int, slot: int) -> int:
        return self.buf.ptrs[owner] + _FLAG_BYTES + slot * self.slot_bytes

    # -- sender --------------------------------------------------------------
    def send(self, obj: Any, first: bool) -> None:
        dev = self.comm.device
        header, tensors = _encode(obj)
        if first or self._header is None or not _same_signature(self._header, header):
            if not first and self._header is not None:
                raise RuntimeError(f"channel {self.tag}: payload signature changed inside a step")
            self._send_header(header, dev)
            self._header = header
            self._ensure_ring(header.metas)
        elif header.leaves != self._header.leaves:
            raise RuntimeError(f"channel {self.tag}: non-tensor values changed between micro-batches")
        lib = _lib.require()
        st = _lib.stream_ptr()
        slot, n = self.seq % RING, self.seq
        if n >= RING:  # the receiver has taken the message that used this slot last
            _lib.check_rc(lib.b200_stream_wait_flag_geq(self._flag(self._me, 1, slot), n - RING + 1, st), "p2p wait free")
        base = self._slot(self._peer, slot)
        for t, off in zip(tensors, self._offsets):
            td = t.detach()
            if not td.is_contiguous():
                td = td.contiguous()
            nbytes = td.numel() * td.element_size()
            _lib.check_rc(lib.b200_copy_async(base + off, td.data_ptr(), nbytes, st), "p2p copy")
            self.bytes_moved += nbytes
        _lib.check_rc(lib.b200_stream_store_flag(self._flag(self._peer, 0, slot), n + 1, st), "p2p signal full")
        self.seq += 1

    def _send_header(self, header, dev) -> None:
        import pickle
        blob = pickle.dumps(header)
        n = torch.tensor([len(blob)], dtype=torch.int64, device=dev)
        dist.send(n, self.dst, group=self.group)
        dist.send(torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(dev), self.dst, group=self.group)

    def flush(self) -> None:
        pass  # copies are stream-ordered; nothing is held on the host

    # -- receiver ------------------------------------------------------------
    def post_recv(self, first: bool) -> None:
        dev = self.comm.device
        if first or self._header is None:
            import pickle
            n = torch.zeros(1, dtype=torch.int64, device=dev)
            dist.recv(n, self.src, group=self.group)
            buf = torch.empty(int(n.item()), dtype=torch.uint8, device=dev)
            dist.recv(buf, self.src, group=self.group)
            self._header = pickle.loads(buf.cpu().numpy().tobytes())
            self._ensure_ring(self._header.metas)
        self._expected += 1

    def wait_recv(self) -> Any:
        if self._expected <= 0:
            raise RuntimeError(f"channel {self.tag}: wait_recv without a posted receive")
        self._expected -= 1
        lib = _lib.require()
        st = _lib.stream_ptr()
        dev = self.comm.device
        slot, n = self.seq % RING, self.seq
        _lib.check_rc(lib.b200_stream_wait_flag_geq(self._flag(self._me, 0, slot), n + 1, st), "p2p wait full")
        base = self._slot(self._me, slot)
        out = []
        for (dtype, shape, rg), off in zip(self._header.metas, self._offsets):
            t = torch.empty(shape, dtype=dtype, device=dev)
            nbytes = t.numel() * t.element_size()
            _lib.check_rc(lib.b200_copy_async(t.data_ptr(), base + off, nbytes, st), "p2p copy out")
            self.bytes_moved += nbytes
            if rg and t.is_floating_point():
                t.requires_grad_(True)
            out.append(t)
        _lib.check_rc(lib.b200_stream_store_flag(self._flag(self._peer, 1, slot), n + 1, st), "p2p signal free")
        self.seq += 1
        return _decode(self._header, out)

    def pending_recvs(self) -> int:
        return self._expected
