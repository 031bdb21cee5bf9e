"""Serving engine: continuous batching over a paged KV cache, tensor parallel inside a replica.

One ``ServingEngine`` per rank of a replica (SPMD: every TP rank sees the same requests and makes the same
scheduling decisions, so no request metadata is exchanged at run time).  A step prefills newly admitted
prompts (one forward per prompt: causal flash attention + page writes) and then decodes one token for
every running sequence (paged decode-attention kernel).  Decode steps are captured in CUDA graphs per
padded batch size, because a 32-layer decode step is launch-bound from Python otherwise.

Reference point: ``Optimus_Inference.generate`` serves a single static batch with a dense cache
(opt_prime/opt_prime/inference.py:916-1120); everything here is the part its design lacks.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..engine import Optimus_p
from ..models.llama import B200LlamaLayer
from .loadgen import summarize
from .paged_kv import PAGE, PagedKVAdaptor, PagedKVCache
from .scheduler import ContinuousBatchingScheduler, Request

_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 96, 128, 192, 256, 384, 512)


class ServingEngine:
    def __init__(self, module: nn.Module, tp_size: int = 1, use_gpu: bool = True, dtype: torch.dtype = torch.bfloat16,
                 num_pages: Optional[int] = None, max_seqs: int = 256, max_seq_len: int = 4096, cuda_graphs: bool = True,
                 kv_memory_fraction: float = 0.85, pool: Optional[torch.Tensor] = None, tp_backend: str = "nccl",
                 max_prefill_per_step: int = 4, dp_size: int = 1):
        if not torch.cuda.is_available() or not use_gpu:
            dtype, cuda_graphs = (torch.float32 if dtype == torch.bfloat16 else dtype), False
        # dp_size > 1: independent replicas inside one job (weights are broadcast from the first replica at set-up)
        self._e = Optimus_p(module, num_mb=1, use_gpu=use_gpu, pp_size=1, dp_size=dp_size, tp_size=tp_size, dtype=dtype,
                            sequence_parallel=False, tp_backend=tp_backend, input_names=["input_ids", "position_ids"],
                            trace_kwargs={"logits_to_keep": 1})
        self._e.eval()
        self.device, self.comm, self.tpl = self._e.device, self._e.comm, self._e.tpl
        self.stage_module = self._e.stage_module
        self.layers: List[B200LlamaLayer] = [m for m in self.stage_module.modules() if isinstance(m, B200LlamaLayer)]
        if not self.layers:
            raise ValueError("the serving engine needs a Llama-family model (fused layers)")
        l0 = self.layers[0]
        self.max_blocks = (max_seq_len + PAGE - 1) // PAGE
        self.max_seqs = max_seqs
        page_bytes = 2 * len(self.layers) * PAGE * l0.hkv * l0.head_dim * torch.empty((), dtype=dtype).element_size()
        if num_pages is None:
            if self.device.type == "cuda":
                free, _ = torch.cuda.mem_get_info(self.device)
                num_pages = max(64, int(free * kv_memory_fraction) // page_bytes)
            else:
                num_pages = 512
            if tp_size > 1 and self.tpl.tp_group is not None:
                # every rank of the replica must see the same pool size: admission decisions depend on it
                import torch.distributed as dist
                n = torch.tensor([num_pages], dtype=torch.int64, device=self.device)
                dist.all_reduce(n, op=dist.ReduceOp.MIN, group=self.tpl.tp_group)
                num_pages = int(n.item())
        first = min(l.layer_idx for l in self.layers)
        self.cache = PagedKVCache(len(self.layers), l0.hkv, l0.head_dim, num_pages, max_seqs, self.max_blocks, dtype, self.device,
                                  pool=pool, layer_offset=first, q_heads=l0.hq)
        self.adaptor = PagedKVAdaptor(self.cache)
        for l in self.layers:
            l.kv_cache = self.adaptor
        self.scheduler = ContinuousBatchingScheduler(self.cache, max_running=max_seqs, max_prefill_per_step=max_prefill_per_step)
        self.use_graphs = cuda_graphs and self.device.type == "cuda"
        self._graphs: Dict[int, dict] = {}
        self.decode_steps = 0
        self.prefill_tokens = 0

    # ---- model calls -------------------------------------------------------------------------------
    @torch.no_grad()
    def _forward(self, ids: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        out, _ = self.stage_module(ids, pos)
        logits = out["logits"] if isinstance(out, dict) else out
        return logits[:, -1, :]

    @torch.no_grad()
    def prefill(self, req: Request) -> int:
        """Run the prompt of ``req`` (already admitted: it has a slot and pages); returns the first generated token."""
        S = req.prompt_len
        ids = torch.tensor(req.prompt, dtype=torch.long, device=self.device).view(1, S)
        pos = torch.arange(S, dtype=torch.long, device=self.device).view(1, S)
        ad = self.adaptor
        ad.mode = "prefill"
        ad.table = self.cache.block_table[req.slot:req.slot + 1]
        ad.seq_idx = torch.zeros(S, dtype=torch.int32, device=self.device)
        ad.seq_lens = None
        logits = self._forward(ids, pos)
        self.prefill_tokens += S
        return int(logits.argmax(-1).item())

    def _bucket(self, n: int) -> int:
        for b in _BUCKETS:
            if b >= n:
                return b
        return n

    def _decode_buffers(self, b: int) -> dict:
        g = self._graphs.get(b)
        if g is None:
            dev = self.device
            g = {"ids": torch.zeros(b, 1, dtype=torch.long, device=dev), "pos": torch.zeros(b, 1, dtype=torch.long, device=dev),
                 "table": torch.zeros(b, self.max_blocks, dtype=torch.int32, device=dev),
                 "lens": torch.ones(b, dtype=torch.int32, device=dev), "seq_idx": torch.arange(b, dtype=torch.int32, device=dev),
                 "out": torch.zeros(b, dtype=torch.long, device=dev), "graph": None, "warm": 0}
            self._graphs[b] = g
        return g

    @torch.no_grad()
    def decode(self, reqs: List[Request]) -> List[int]:
        """One token for every request in ``reqs`` (all running, each with >= 1 generated token)."""
        n = len(reqs)
        b = self._bucket(n) if self.use_graphs else n
        g = self._decode_buffers(b)
        slots = torch.tensor([r.slot for r in reqs], dtype=torch.long)
        last = torch.tensor([r.generated[-1] for r in reqs], dtype=torch.long)
        posv = torch.tensor([r.total_len - 1 for r in reqs], dtype=torch.long)
        for r in reqs:
            self.cache.ensure_capacity(r.slot, r.total_len)
        if b > n:  # padded slots read and write the reserved scratch page 0
            g["ids"][n:].zero_()
            g["pos"][n:].zero_()
            g["table"][n:].zero_()
            g["lens"][n:].fill_(1)
        g["ids"][:n, 0].copy_(last, non_blocking=True)
        g["pos"][:n, 0].copy_(posv, non_blocking=True)
        g["lens"][:n].copy_((posv + 1).to(torch.int32), non_blocking=True)
        g["table"][:n].copy_(self.cache.block_table.index_select(0, slots.to(self.device)))
        ad = self.adaptor
        ad.mode, ad.table, ad.seq_idx, ad.seq_lens = "decode", g["table"], g["seq_idx"], g["lens"]

        def body():
            g["out"].copy_(self._forward(g["ids"], g["pos"]).argmax(-1))

        if not self.use_graphs:
            body()
        elif g["graph"] is None:
            body()  # warm-up runs outside capture (lazy initialisation, kernel attribute set-up)
            g["warm"] += 1
            if g["warm"] >= 2:
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    body()
                g["graph"] = graph
        else:
            g["graph"].replay()
        self.decode_steps += 1
        return g["out"][:n].tolist()

    def warmup(self, max_batch: Optional[int] = None, prompt_len: int = 256) -> None:
        """Run one prefill and capture the decode graphs for every batch bucket up to ``max_batch`` (untimed set-up)."""
        max_batch = max_batch or self.max_seqs
        reqs = []
        for i in range(min(max_batch, self.max_seqs)):
            r = Request(rid=-1 - i, prompt=[1] * (prompt_len if i == 0 else 4), max_new_tokens=4)
            if not self.cache.can_admit(r.prompt_len + 8):
                break
            r.slot = self.cache.add_sequence(r.prompt_len + 8)
            r.generated = [self.prefill(r)] if i == 0 else [1]
            self.cache.seq_len[r.slot] = r.prompt_len
            reqs.append(r)
        for b in _BUCKETS:
            if b > len(reqs):
                break
            for _ in range(3 if self.use_graphs else 1):  # two eager runs, then the capture
                self.decode(reqs[:b])
        for r in reqs:
            self.cache.free_sequence(r.slot)
        self.decode_steps = 0
        self.prefill_tokens = 0
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    # ---- request loop ------------------------------------------------------------------------------------
    def serve(self, requests: List[Request], realtime: bool = True, max_wall_s: Optional[float] = None) -> Dict[str, float]:
        """Run ``requests`` to completion.  With ``realtime`` arrivals follow the wall clock; otherwise the clock
        jumps to the next arrival whenever the engine is idle (fast simulation)."""
        sch = self.scheduler
        for r in sorted(requests, key=lambda r: r.arrival_s):
            sch.add_request(r)
        t0 = time.perf_counter()
        skew = 0.0

        def now():
            return time.perf_counter() - t0 + skew

        def group_now():
            """The clock every scheduling decision uses: the first tensor-parallel rank's, broadcast to the group, so
            that all ranks of a replica admit the same requests in the same step (their own clocks differ by
            microseconds, which is enough to split a batch differently and mismatch the collectives)."""
            t = now()
            if self.tpl.tp_size > 1 and self.tpl.tp_group is not None:
                import torch.distributed as dist
                buf = torch.tensor([t], dtype=torch.float64, device=self.device)
                dist.broadcast(buf, src=self.tpl.tp_ranks()[0], group=self.tpl.tp_group)
                t = float(buf.item())
            return t

        while sch.has_work():
            t_step = group_now()
            plan = sch.plan_step(t_step)
            if not plan.prefill and not plan.decode:
                nxt = sch.waiting[0].arrival_s if sch.waiting else None
                if nxt is None:
                    break
                wait = nxt - t_step
                if wait > 0:
                    if realtime:
                        time.sleep(min(wait, 0.01))
                    else:
                        skew += wait
                continue
            for req in plan.prefill:
                tok = self.prefill(req)
                sch.after_prefill(req, tok, now())
            if plan.decode:
                toks = self.decode(plan.decode)
                sch.after_decode(plan.decode, toks, now())
            if max_wall_s is not None and t_step > max_wall_s:
                break
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        wall = now()
        m = summarize(sch.finished, wall)
        m.update({"decode_steps": self.decode_steps, "prefill_tokens": self.prefill_tokens, "peak_running": sch.peak_running,
                  "kv_pages": self.cache.num_pages, "unfinished": len(sch.running) + len(sch.waiting)})
        return m
