"""Prefill/decode-disaggregated serving: prefill GPUs run prompts, decode GPUs run continuous batching.

A *pair* is one prefill rank and one decode rank that share symmetric KV page pools (``serve/pd.py``).  Requests are
dealt round-robin to the pairs.  Inside a pair:

1. the decode worker admits a request when it has arrived and pages are free, reserves the pages in ITS pool and posts
   the destination page list into a mailbox in the prefill rank's memory;
2. the prefill worker takes requests in arrival order, runs the prompt into scratch pages of its own pool (causal flash
   attention + page writes), reads the destination list, and launches ``b200_kv_push``: the pages cross NVLink by
   peer stores and the request's ready word on the decode rank is raised to ``first_token + 1`` after the data;
3. the decode worker polls the ready words of its pending requests between decode steps, moves ready requests into the
   running batch and decodes one token per step for all of them (CUDA-graph replay, paged decode attention).

Decode steps therefore never wait behind a prompt, and TTFT is prefill time plus one page push.  The transport is an
interface: :class:`LoopbackTransport` moves pages inside one process (CPU tests of the protocol),
:class:`PeerTransport` is the NVLink path.  The reference has no disaggregated serving (its cache is a dense
per-process tensor, opt_prime/opt_prime/kv_cache.py:19-254).
"""
from __future__ import annotations

import collections
import time
from typing import Deque, Dict, List, Optional

import torch

from .loadgen import summarize
from .scheduler import Request

MAILBOX_SLOTS = 1024


# ------------------------------------------------------------------------------------------------ transports
class LoopbackTransport:
    """Both workers live in this process; a push is a tensor copy between the two caches' pools."""

    def __init__(self, prefill_cache, decode_cache):
        self.src, self.dst = prefill_cache, decode_cache
        self._pages: Dict[int, List[int]] = {}
        self._ready: Dict[int, int] = {}
        self.bytes_pushed = 0

    def post_dst_pages(self, rid: int, pages: List[int]) -> None:
        self._pages[rid] = list(pages)

    def poll_dst_pages(self, rid: int) -> Optional[List[int]]:
        return self._pages.pop(rid, None)

    def push(self, rid: int, src_pages: List[int], dst_pages: List[int], token: int) -> None:
        s = torch.tensor(src_pages, dtype=torch.long, device=self.src.pool.device)
        d = torch.tensor(dst_pages, dtype=torch.long, device=self.dst.pool.device)
        self.dst.pool[:, :, d] = self.src.pool[:, :, s].to(self.dst.pool.device)
        self.bytes_pushed += self.src.pool[:, :, s].numel() * self.src.pool.element_size()
        self._ready[rid] = token

    def poll_ready(self, rids) -> Dict[int, int]:
        out = {r: self._ready.pop(r) for r in list(rids) if r in self._ready}
        return out


class PeerTransport:
    """NVLink path between the two ranks of ``group``: symmetric page pools, ready words and a page-list mailbox."""

    def __init__(self, group, device, layers: int, pool_pages: int, page_bytes: int, max_blocks: int, is_prefill: bool):
        from ..ops import _lib
        from ..parallel.symm import SymmetricBuffer
        from .pd import KVPagePusher
        self._lib = _lib
        self.device = device
        self.is_prefill = is_prefill
        self.pusher = KVPagePusher(group, device, layers, pool_pages, page_bytes, request_slots=MAILBOX_SLOTS)
        self.row = 2 + max_blocks   # [sequence number, n_pages, page ids ...]
        self.mail = SymmetricBuffer(group, MAILBOX_SLOTS * self.row * 4, device)
        self.rank, self.peer = self.pusher.rank, 1 - self.pusher.rank
        self.mail_local = self.mail.view(torch.int32, MAILBOX_SLOTS * self.row).view(MAILBOX_SLOTS, self.row)
        self._stage = torch.zeros(self.row, dtype=torch.int32, device=device)
        self._host = torch.zeros(self.row, dtype=torch.int32).pin_memory()

    @property
    def pool_bytes(self) -> torch.Tensor:
        return self.pusher.pool.local

    @property
    def bytes_pushed(self) -> int:
        return self.pusher.bytes_pushed

    # decode side ----------------------------------------------------------------------------------------
    def post_dst_pages(self, rid: int, pages: List[int]) -> None:
        lib = self._lib.require()
        slot = rid % MAILBOX_SLOTS
        self._host.zero_()
        self._host[1] = len(pages)
        self._host[2:2 + len(pages)] = torch.tensor(pages, dtype=torch.int32)
        self._stage.copy_(self._host, non_blocking=True)
        st = self._lib.stream_ptr()
        dst = self.mail.ptrs[self.peer] + slot * self.row * 4
        # the page list first, then the sequence number that publishes it (stream order + system-scope release store)
        self._lib.check_rc(lib.b200_copy_async(dst + 4, self._stage.data_ptr() + 4, (self.row - 1) * 4, st), "pd mailbox")
        self._lib.check_rc(lib.b200_stream_store_flag(dst, rid + 1, st), "pd mailbox flag")
        torch.cuda.current_stream().synchronize()  # `_stage` is reused by the next post

    def poll_ready(self, rids) -> Dict[int, int]:
        rids = list(rids)
        if not rids:
            return {}
        idx = torch.tensor([r % MAILBOX_SLOTS for r in rids], dtype=torch.long, device=self.device)
        vals = self.pusher.ready_words.index_select(0, idx).tolist()
        out = {}
        for r, v in zip(rids, vals):
            if v > 0:
                out[r] = v - 1
                self.pusher.clear_ready(r % MAILBOX_SLOTS)
        return out

    # prefill side ---------------------------------------------------------------------------------------
    def poll_dst_pages(self, rid: int) -> Optional[List[int]]:
        row = self.mail_local[rid % MAILBOX_SLOTS].tolist()
        if row[0] != rid + 1:
            return None
        return row[2:2 + row[1]]

    def push(self, rid: int, src_pages: List[int], dst_pages: List[int], token: int) -> None:
        self.pusher.push(self.peer, torch.tensor(src_pages, dtype=torch.int32), torch.tensor(dst_pages, dtype=torch.int32),
                         request_slot=rid % MAILBOX_SLOTS, ready_value=token + 1)


# ------------------------------------------------------------------------------------------------ workers
class PrefillWorker:
    def __init__(self, engine, transport, requests: List[Request]):
        self.e, self.t = engine, transport
        self.queue: Deque[Request] = collections.deque(sorted(requests, key=lambda r: r.arrival_s))
        self.current: Optional[tuple] = None   # (request, first token, local slot) waiting for its destination pages
        self.done = 0

    def has_work(self) -> bool:
        return bool(self.queue) or self.current is not None

    def step(self, now: float) -> bool:
        """Advance by at most one prompt; returns False when there was nothing to do yet."""
        cache = self.e.cache
        if self.current is None:
            if not self.queue or self.queue[0].arrival_s > now:
                return False
            req = self.queue.popleft()
            slot = cache.add_sequence(req.prompt_len)
            shadow = Request(rid=req.rid, prompt=req.prompt, max_new_tokens=1)
            shadow.slot = slot
            tok = self.e.prefill(shadow)
            self.current = (req, tok, slot)
        req, tok, slot = self.current
        dst = self.t.poll_dst_pages(req.rid)
        if dst is None:
            return False
        n = cache.pages_needed(req.prompt_len)
        self.t.push(req.rid, cache.seq_pages[slot][:n], dst[:n], tok)
        cache.free_sequence(slot)   # later prompts are launched after the push on the same stream
        self.current = None
        self.done += 1
        return True


class DecodeWorker:
    def __init__(self, engine, transport, requests: List[Request], max_running: int = 256):
        self.e, self.t = engine, transport
        self.waiting: Deque[Request] = collections.deque(sorted(requests, key=lambda r: r.arrival_s))
        self.pending: Dict[int, Request] = {}
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self.max_running = max_running
        self.peak_running = 0

    def has_work(self) -> bool:
        return bool(self.waiting or self.pending or self.running)

    def step(self, now: float) -> bool:
        cache = self.e.cache
        did = False
        while self.waiting and self.waiting[0].arrival_s <= now and len(self.pending) + len(self.running) < self.max_running:
            req = self.waiting[0]
            budget = req.prompt_len + req.max_new_tokens
            if not cache.can_admit(budget):
                break
            self.waiting.popleft()
            req.slot = cache.add_sequence(budget)
            req.t_admitted = now
            self.t.post_dst_pages(req.rid, cache.seq_pages[req.slot][:cache.pages_needed(req.prompt_len)])
            self.pending[req.rid] = req
            did = True
        for rid, tok in self.t.poll_ready(self.pending.keys()).items():
            req = self.pending.pop(rid)
            req.generated.append(tok)
            req.t_first_token = now
            cache.seq_len[req.slot] = req.prompt_len
            if req.is_finished():
                self._finish(req, now)
            else:
                self.running.append(req)
                self.peak_running = max(self.peak_running, len(self.running))
            did = True
        if self.running:
            batch = list(self.running)
            toks = self.e.decode(batch)
            for req, tok in zip(batch, toks):
                req.generated.append(tok)
                cache.seq_len[req.slot] = req.total_len - 1
                if req.is_finished():
                    self._finish(req, now)
            did = True
        return did

    def _finish(self, req: Request, now: float) -> None:
        req.t_finished = now
        if req in self.running:
            self.running.remove(req)
        self.e.cache.free_sequence(req.slot)
        req.slot = -1
        self.finished.append(req)


def run_worker(worker, realtime: bool = True, max_wall_s: Optional[float] = None) -> float:
    """Drive one worker until it has no work left; returns the wall time of the loop."""
    t0 = time.perf_counter()
    while worker.has_work():
        now = time.perf_counter() - t0
        if not worker.step(now) and realtime:
            time.sleep(0.0005)
        if max_wall_s is not None and now > max_wall_s:
            break
    return time.perf_counter() - t0


# ------------------------------------------------------------------------------------------------ multi-rank driver
def run_pd_serving(module, requests: List[Request], n_prefill: int, n_decode: int, max_seqs: int = 256, max_seq_len: int = 4096,
                   prefill_pool_pages: int = 1024, decode_pool_pages: Optional[int] = None, max_wall_s: Optional[float] = None
                   ) -> Optional[Dict[str, float]]:
    """SPMD entry point for ``n_prefill + n_decode`` ranks of one node (``n_prefill == n_decode`` pairs).

    Every rank builds a full replica (tensor parallel size 1), joins its pair's 2-rank group, and runs its role.
    Rank 0 returns the aggregate metrics (decode tokens/s summed over the pairs, TTFT percentiles over all requests)."""
    import torch.distributed as dist

    from .engine import ServingEngine
    from .paged_kv import PAGE
    if n_prefill != n_decode:
        raise ValueError("prefill and decode ranks are paired one to one")
    world, rank = dist.get_world_size(), dist.get_rank()
    if world != n_prefill + n_decode:
        raise ValueError("world size must equal n_prefill + n_decode")
    is_prefill = rank < n_prefill
    pair = rank if is_prefill else rank - n_prefill
    groups = [dist.new_group(ranks=[i, n_prefill + i]) for i in range(n_prefill)]
    cfg = module.config
    layers, hkv = cfg.num_hidden_layers, cfg.num_key_value_heads
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    page_bytes = PAGE * hkv * head_dim * 2
    device = torch.device("cuda", torch.cuda.current_device())
    if decode_pool_pages is None:
        free, _ = torch.cuda.mem_get_info(device)
        weights = sum(p.numel() for p in module.parameters()) * 2
        decode_pool_pages = max(prefill_pool_pages, int((free - weights) * 0.8) // (2 * layers * page_bytes))
    pool_pages = decode_pool_pages   # symmetric buffers have one size; the prefill rank uses the first pages only
    max_blocks = (max_seq_len + PAGE - 1) // PAGE
    transport = PeerTransport(groups[pair], device, layers, pool_pages, page_bytes, max_blocks, is_prefill)
    eng = ServingEngine(module, tp_size=1, dp_size=world, max_seqs=max_seqs, max_seq_len=max_seq_len, num_pages=pool_pages,
                        pool=transport.pool_bytes, cuda_graphs=not is_prefill)
    mine = requests[pair::n_prefill]
    if is_prefill:
        worker = PrefillWorker(eng, transport, mine)
        eng.warmup(max_batch=1)
    else:
        worker = DecodeWorker(eng, transport, mine, max_running=max_seqs)
        eng.warmup()
    dist.barrier()
    wall = run_worker(worker, realtime=True, max_wall_s=max_wall_s)
    torch.cuda.synchronize()
    from ..ops import check_errors
    check_errors()
    local = None
    if not is_prefill:
        local = {"finished": [(r.arrival_s, r.t_first_token, r.t_finished, len(r.generated)) for r in worker.finished], "wall": wall,
                 "peak_running": worker.peak_running, "decode_steps": eng.decode_steps}
    else:
        local = {"prefill_tokens": eng.prefill_tokens, "bytes_pushed": transport.bytes_pushed, "wall": wall}
    gathered: List[Optional[dict]] = [None] * world
    dist.all_gather_object(gathered, local)
    if rank != 0:
        return None
    fin: List[Request] = []
    for g in gathered[n_prefill:]:
        for (arr, tf, te, n) in g["finished"]:
            r = Request(rid=len(fin), prompt=[], max_new_tokens=n, arrival_s=arr)
            r.generated = [0] * n
            r.t_first_token, r.t_finished = tf, te
            fin.append(r)
    wall_all = max(g["wall"] for g in gathered[n_prefill:])
    m = summarize(fin, wall_all)
    m.update({"pairs": n_prefill, "kv_bytes_pushed": sum(g["bytes_pushed"] for g in gathered[:n_prefill]),
              "prefill_tokens": sum(g["prefill_tokens"] for g in gathered[:n_prefill]),
              "peak_running": max(g["peak_running"] for g in gathered[n_prefill:]), "kv_pages": pool_pages,
              "unfinished": len(requests) - len(fin)})
    return m
