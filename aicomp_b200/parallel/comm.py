"""Process-group bring-up and point-to-point transport between pipeline stages.

Capability parity with the reference ``Comm`` (opt_prime/opt_prime/comm.py:19-324):
reads the torchrun environment, initialises ``torch.distributed`` with NCCL on
GPUs or gloo on CPUs over a TCP rendezvous, always creates a world-wide gloo
side group for host-side barriers and object exchange, seeds the RNG with 42,
and can move arbitrary nested Python/tensor objects between ranks
(``send_data`` / ``receive_data``).

The transport itself is redesigned.  The reference sends five blocking messages
per tensor on every micro-batch; here a *channel* between two adjacent stages
exchanges one pickled header per training step (dtypes, shapes,
``requires_grad`` flags, non-tensor leaves, tree structure), after which the
tensor payloads move with non-blocking ``isend``/``irecv`` into cached receive
buffers.  Forward traffic (activations) and backward traffic (gradients) use
separate 2-rank groups, hence separate NCCL communicators and streams, so
posting a receive early can never queue in front of the matching send of the
opposite direction.
"""
from __future__ import annotations

import io
import os
import pickle
from dataclasses import dataclass
from datetime import timedelta
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch.utils import _pytree as pytree

from ..utils.log import get_logger

log = get_logger(__name__)

__all__ = ["Comm", "Channel"]


class _TensorSlot:
    """Placeholder for a tensor leaf inside a pickled header."""

    __slots__ = ("index",)

    def __init__(self, index: int):
        self.index = index

    def __eq__(self, other):
        return isinstance(other, _TensorSlot) and other.index == self.index

    def __hash__(self):
        return hash(("slot", self.index))


@dataclass
class _Header:
    spec: Any                      # pytree spec of the payload
    leaves: List[Any]              # non-tensor leaves in place, _TensorSlot for tensors
    metas: List[Tuple[torch.dtype, Tuple[int, ...], bool]]  # dtype, shape, requires_grad per tensor


class Comm:
    def __init__(self, use_gpu: bool = True, timeout_s: float = 1800.0, seed: int = 42):
        torch.manual_seed(seed)
        self.rank = int(os.environ.get("RANK", "0"))
        self.world_size = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.local_world_size = int(os.environ.get("LOCAL_WORLD_SIZE", "1"))
        self.master_addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        self.master_port = os.environ.get("MASTER_PORT", "29500")
        self.use_gpu = bool(use_gpu) and torch.cuda.is_available()
        if use_gpu and not torch.cuda.is_available():
            log.warning("use_gpu=True but no CUDA device is visible; running on CPU with gloo")
        self.backend = "nccl" if self.use_gpu else "gloo"
        if self.use_gpu:
            n = torch.cuda.device_count()
            if self.local_rank >= n:
                raise RuntimeError(f"local_rank {self.local_rank} has no GPU (visible: {n}); one process per GPU is required")
            torch.cuda.set_device(self.local_rank)
            self.device = torch.device("cuda", self.local_rank)
        else:
            self.device = torch.device("cpu")
        self.host_group = None  # gloo group spanning the world (barriers, object exchange)
        self._pair_groups: Dict[Tuple[int, int, str], Any] = {}
        if self.world_size > 1:
            if not dist.is_initialized():
                kwargs = {}
                if self.use_gpu:
                    kwargs["device_id"] = self.device
                dist.init_process_group(backend=self.backend, rank=self.rank, world_size=self.world_size,
                                        init_method=f"tcp://{self.master_addr}:{self.master_port}",
                                        timeout=timedelta(seconds=timeout_s), **kwargs)
            if self.backend == "gloo":
                self.host_group = dist.group.WORLD
            else:
                self.host_group = dist.new_group(backend="gloo", timeout=timedelta(seconds=timeout_s))

    # ------------------------------------------------------------------ basics
    def barrier(self) -> None:
        """Host-side barrier over the gloo group (safe when several ranks share a GPU)."""
        if self.world_size > 1:
            dist.barrier(group=self.host_group)

    def new_group(self, ranks: List[int], backend: Optional[str] = None):
        """Collective: every rank must call with the same arguments in the same order."""
        if self.world_size == 1:
            return None
        return dist.new_group(ranks=ranks, backend=backend or self.backend)

    def broadcast_object(self, obj: Any, src: int = 0) -> Any:
        if self.world_size == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self.host_group)
        return box[0]

    def all_gather_object(self, obj: Any) -> List[Any]:
        if self.world_size == 1:
            return [obj]
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.host_group)
        return out

    # ------------------------------------------------------------------ blocking object transport
    def send_data(self, obj: Any, to_rank: int, device=None, group=None) -> None:
        """Blocking send of any nested structure of tensors / Python values."""
        header, tensors = _encode(obj)
        blob = pickle.dumps(header)
        dev = self.device
        n = torch.tensor([len(blob)], dtype=torch.int64, device=dev)
        dist.send(n, to_rank, group=group)
        dist.send(torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(dev), to_rank, group=group)
        for t in tensors:
            dist.send(t.detach().contiguous().to(dev), to_rank, group=group)

    def receive_data(self, from_rank: int, device=None, group=None) -> Any:
        dev = self.device
        n = torch.zeros(1, dtype=torch.int64, device=dev)
        dist.recv(n, from_rank, group=group)
        buf = torch.empty(int(n.item()), dtype=torch.uint8, device=dev)
        dist.recv(buf, from_rank, group=group)
        header: _Header = pickle.loads(buf.cpu().numpy().tobytes())
        tensors = []
        for dtype, shape, rg in header.metas:
            t = torch.empty(shape, dtype=dtype, device=dev)
            dist.recv(t, from_rank, group=group)
            tensors.append(t)
        return _decode(header, tensors)

    # ------------------------------------------------------------------ channels
    def make_channel(self, src: int, dst: int, tag: str, group=None, backend: str = "nccl") -> "Channel":
        """``backend='peer'``: ring in the receiver's memory written by the sender's copy engines (one node, CUDA);
        ``'nccl'``: ``isend``/``irecv`` of the process group (any backend, any topology)."""
        if backend == "peer":
            from .p2p import PeerChannel
            return PeerChannel(self, src, dst, tag, group)
        return Channel(self, src, dst, tag, group)


def _encode(obj: Any) -> Tuple[_Header, List[torch.Tensor]]:
    leaves, spec = pytree.tree_flatten(obj)
    tensors: List[torch.Tensor] = []
    out_leaves: List[Any] = []
    metas = []
    for leaf in leaves:
        if isinstance(leaf, torch.Tensor):
            out_leaves.append(_TensorSlot(len(tensors)))
            metas.append((leaf.dtype, tuple(leaf.shape), bool(leaf.requires_grad)))
            tensors.append(leaf)
        else:
            out_leaves.append(leaf)
    return _Header(spec, out_leaves, metas), tensors


def _decode(header: _Header, tensors: List[torch.Tensor]) -> Any:
    leaves = [tensors[l.index] if isinstance(l, _TensorSlot) else l for l in header.leaves]
    return pytree.tree_unflatten(leaves, header.spec)


class Channel:
    """One direction of traffic between two ranks (``src`` -> ``dst``).

    ``send(obj, first)`` / ``post_recv(first)`` + ``wait_recv()``: with
    ``first=True`` a header precedes the payload and replaces the cached one;
    otherwise the cached header is reused and only tensors move.  Payload sends
    and receives are non-blocking; ``flush()`` waits for outstanding sends.
    """

    def __init__(self, comm: Comm, src: int, dst: int, tag: str, group=None):
        self.comm = comm
        self.src, self.dst, self.tag = src, dst, tag
        self.group = group
        self.is_sender = comm.rank == src
        self.is_receiver = comm.rank == dst
        self._header: Optional[_Header] = None
        self._pending_sends: List[Tuple[Any, Any]] = []
        self._recv_queue: List[Tuple[List[Any], List[torch.Tensor]]] = []
        self._buffers: Dict[int, List[List[torch.Tensor]]] = {}
        self._buf_rr = 0
        self.bytes_moved = 0

    # -- sender ----------------------------------------------------------
    def send(self, obj: Any, first: bool) -> None:
        dev = self.comm.device
        header, tensors = _encode(obj)
        if first or self._header is None or not _same_signature(self._header, header):
            if not first and self._header is not None:
                raise RuntimeError(f"channel {self.tag}: payload signature changed inside a step")
            blob = pickle.dumps(header)
            n = torch.tensor([len(blob)], dtype=torch.int64, device=dev)
            dist.send(n, self.dst, group=self.group)
            dist.send(torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(dev), self.dst, group=self.group)
            self._header = header
        elif any(not isinstance(l, _TensorSlot) for l in header.leaves) and header.leaves != self._header.leaves:
            raise RuntimeError(f"channel {self.tag}: non-tensor values changed between micro-batches")
        for t in tensors:
            td = t.detach()
            if not td.is_contiguous():
                td = td.contiguous()
            if td.device != dev:
                td = td.to(dev)
            work = dist.isend(td, self.dst, group=self.group)
            self._pending_sends.append((work, td))
            self.bytes_moved += td.numel() * td.element_size()

    def flush(self) -> None:
        for work, _ in self._pending_sends:
            work.wait()
        self._pending_sends.clear()

    # -- receiver --------------------------------------------------------
    def post_recv(self, first: bool) -> None:
        dev = self.comm.device
        if first or self._header is None:
            n = torch.zeros(1, dtype=torch.int64, device=dev)
            dist.recv(n, self.src, group=self.group)
            buf = torch.empty(int(n.item()), dtype=torch.uint8, device=dev)
            dist.recv(buf, self.src, group=self.group)
            self._header = pickle.loads(buf.cpu().numpy().tobytes())
        bufs = [torch.empty(shape, dtype=dtype, device=dev) for dtype, shape, _ in self._header.metas]
        works = [dist.irecv(t, self.src, group=self.group) for t in bufs]
        self._recv_queue.append((works, bufs))

    def wait_recv(self) -> Any:
        works, bufs = self._recv_queue.pop(0)
        for w in works:
            w.wait()
        assert self._header is not None
        for t, (_, _, rg) in zip(bufs, self._header.metas):
            self.bytes_moved += t.numel() * t.element_size()
            if rg and t.is_floating_point():
                t.requires_grad_(True)
        return _decode(self._header, bufs)

    def pending_recvs(self) -> int:
        return len(self._recv_queue)


def _same_signature(a: _Header, b: _Header) -> bool:
    if a.metas != b.metas or a.spec != b.spec:
        return False
    for x, y in zip(a.leaves, b.leaves):
        tx, ty = isinstance(x, _TensorSlot), isinstance(y, _TensorSlot)
        if tx != ty:
            return False
    return True
