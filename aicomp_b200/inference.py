"""``Optimus_Inference``: pipeline / tensor-parallel autoregressive generation.

Constructor keywords and methods follow the reference (opt_prime/opt_prime/inference.py:91-1226):
three KV modes (no cache: recompute the whole sequence per token; internal cache per attention module;
external ``KVCacheManager``), ``generate`` with greedy / temperature / top-k / top-p sampling and an
optional streamer, the explicit prefill/decode API through
:class:`~aicomp_b200.parallel.schedule_infer.ScheduleGeneration`, LoRA loading/merging, and an MPS-safe
``barrier``.  Fixed relative to the reference: decode batches keep shape ``[B, 1]``, the cache stores GQA
heads, generation stops early once every sequence has produced EOS, and the next token travels from the
last to the first stage in one small broadcast over the pipeline group per step (the reference does two
P2P round trips and two TP broadcasts per token, inference.py:1002-1098).  Continuous batching with a
paged cache is the job of :mod:`aicomp_b200.serve`.
"""
from __future__ import annotations

from typing import Any, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .engine import IR_Anal, Optimus_p
from .kv_cache import CachedScaledDotProductAttention, DenseKVAdaptor, KVCacheManager
from .parallel.schedule_infer import ScheduleGeneration, ScheduleInference

__all__ = ["Optimus_Inference", "sample_token"]


def sample_token(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 50, top_p: float = 0.95, do_sample: bool = True
                 ) -> torch.Tensor:
    """Next token per row of ``logits [B, V]``: argmax, or a draw after temperature, top-k and nucleus filtering."""
    if not do_sample:
        return logits.argmax(dim=-1)
    logits = logits.float()
    if temperature and temperature != 1.0:
        logits = logits / temperature
    if top_k and top_k > 0:
        k = min(int(top_k), logits.shape[-1])
        kth = torch.topk(logits, k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and top_p < 1.0:
        s_logits, s_idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.softmax(s_logits, dim=-1).cumsum(-1)
        drop = cum > top_p
        drop[..., 1:] = drop[..., :-1].clone()  # keep the first token that crosses the threshold
        drop[..., 0] = False
        logits = logits.masked_fill(torch.zeros_like(drop).scatter(-1, s_idx, drop), float("-inf"))
    return torch.multinomial(torch.softmax(logits, dim=-1), 1).squeeze(-1)


class Optimus_Inference:
    def __init__(self, module: nn.Module, use_gpu: bool = True, pp_size: int = 1, dp_size: int = 1, tp_size: int = 1,
                 max_batch_size: int = 32, max_seq_len: int = 2048, dtype: torch.dtype = torch.bfloat16,
                 ir_analyze: IR_Anal = IR_Anal.PARALLEL, use_kv_cache: bool = False, serving_mode: bool = False,
                 use_kv_manager: bool = False, dynamo_capture: bool = False, use_mps: bool = False, partitioner: str = "auto",
                 fused_kernels: Optional[bool] = None, tp_backend: str = "nccl"):
        if not use_gpu or not torch.cuda.is_available():
            dtype = torch.float32 if dtype == torch.bfloat16 and not torch.cuda.is_available() else dtype
        self.use_kv_cache = use_kv_cache or use_kv_manager
        self.use_kv_manager = use_kv_manager
        self.serving_mode = serving_mode
        self.use_mps = use_mps
        self.max_batch_size, self.max_seq_len = max_batch_size, max_seq_len
        input_names = ["input_ids", "position_ids"] if self.use_kv_cache else None
        self._e = Optimus_p(module, num_mb=1, use_gpu=use_gpu, pp_size=pp_size, dp_size=dp_size, tp_size=tp_size,
                            ir_analyze=ir_analyze, dynamo_capture=dynamo_capture, partitioner=partitioner, dtype=dtype,
                            fused_kernels=fused_kernels, sequence_parallel=False, tp_backend=tp_backend, input_names=input_names)
        e = self._e
        e.eval()
        self.comm, self.tpl, self.device, self.plan = e.comm, e.tpl, e.device, e.plan
        self.stage_module = e.stage_module
        self.fwd_in, self.fwd_out = e.fwd_in, e.fwd_out
        self.dtype = dtype
        self.model_config = e.model_config
        self._schedule_infer: Optional[ScheduleInference] = None
        self._schedule_gen: Optional[ScheduleGeneration] = None
        self.kv_manager: Optional[KVCacheManager] = None
        self._cached_sdpa_modules: List[CachedScaledDotProductAttention] = []
        self._adaptors: List[DenseKVAdaptor] = []
        if self.use_kv_cache:
            self._inject_kv_cache_into_graph()

    # ---- plumbing shared with the schedules --------------------------------------------------
    def _to_device(self, t: torch.Tensor) -> torch.Tensor:
        return self._e._to_device(t)

    def _share_int(self, v: Optional[int]) -> int:
        """Value known on the first stage, needed on all stages of this pipeline (e.g. prompt length)."""
        if self.tpl.pp_size == 1:
            return int(v)
        t = torch.tensor([v if v is not None else 0], dtype=torch.int64, device=self.device)
        dist.broadcast(t, src=self.tpl.get_first_rank(), group=self.tpl.pp_group)
        return int(t.item())

    # ---- KV cache wiring ------------------------------------------------------------------------
    def _fused_layers(self):
        from .models.llama import B200LlamaLayer
        return [m for m in self.stage_module.modules() if isinstance(m, B200LlamaLayer)]

    def _inject_kv_cache_into_graph(self) -> None:
        """Generic graphs: swap every SDPA call for a caching module (the reference does this on the FX graph too,
        inference.py:845-913).  Fused Llama layers take a cache adaptor instead (set in ``init_kv_cache``)."""
        import torch.nn.functional as F
        g = self.stage_module.graph
        idx = 0
        for node in list(g.nodes):
            if node.op == "call_function" and node.target in (F.scaled_dot_product_attention, torch._C._nn.scaled_dot_product_attention):
                name = f"cached_sdpa_{idx}"
                mod = CachedScaledDotProductAttention(idx, self.max_batch_size, self.max_seq_len)
                self.stage_module.add_module(name, mod)
                with g.inserting_after(node):
                    new = g.call_module(name, node.args, dict(node.kwargs))
                node.replace_all_uses_with(new)
                g.erase_node(node)
                self._cached_sdpa_modules.append(mod)
                idx += 1
        if idx:
            self.stage_module.recompile()
        if not self._fused_layers() and not self._cached_sdpa_modules and self.tpl.is_first_stage():
            pass  # a stage without attention (e.g. embedding only) has nothing to cache

    def init_kv_cache(self, num_layers: Optional[int] = None, num_heads: Optional[int] = None, head_dim: Optional[int] = None,
                      batch_size: Optional[int] = None, max_seq_len: Optional[int] = None) -> KVCacheManager:
        layers = self._fused_layers()
        if layers:
            first = min(l.layer_idx for l in layers)
            n = max(l.layer_idx for l in layers) - first + 1
            heads, hd = layers[0].hkv, layers[0].head_dim
        else:
            first, n = 0, len(self._cached_sdpa_modules)
            heads, hd = num_heads, head_dim
            if n and (heads is None or hd is None):
                raise ValueError("num_heads and head_dim are required for models without fused layers")
        self.kv_manager = KVCacheManager(max(n, 0), heads or 1, hd or 1, self.max_batch_size, max_seq_len or self.max_seq_len,
                                         self.dtype, self.device, layer_offset=first)
        self.kv_manager.allocate(batch_size)
        self._attach_kv_manager()
        return self.kv_manager

    def _attach_kv_manager(self) -> None:
        if self.kv_manager is None:
            return
        self._adaptors = []
        for l in self._fused_layers():
            ad = DenseKVAdaptor(self.kv_manager)
            l.kv_cache = ad
            self._adaptors.append(ad)
        for m in self._cached_sdpa_modules:
            m.attach(self.kv_manager)
            m.enable()

    def _ensure_cache(self, batch: int) -> None:
        if self.kv_manager is None or not self.kv_manager.is_allocated:
            self.init_kv_cache(batch_size=batch)
        for m in self._cached_sdpa_modules:
            m.enable()

    def _advance_cache(self, n: int) -> None:
        if self.kv_manager is not None:
            self.kv_manager.advance(n)

    def clear_kv_cache(self) -> None:
        if self.kv_manager is not None:
            self.kv_manager.clear()
        for m in self._cached_sdpa_modules:
            m.clear()

    def free_kv_cache(self) -> None:
        if self.kv_manager is not None:
            self.kv_manager.free()
        for m in self._cached_sdpa_modules:
            m.free()

    def release_kv_cache(self) -> None:
        self.free_kv_cache()
        for l in self._fused_layers():
            l.kv_cache = None
        self.kv_manager = None

    # ---- simple API -----------------------------------------------------------------------------------
    def eval(self):
        self._e.eval()
        return self

    def train(self, mode: bool = False):
        self._e.train(mode)
        return self

    def parameters(self):
        return self.stage_module.parameters()

    def is_first_stage(self) -> bool:
        return self.tpl.is_first_stage()

    def is_last_stage(self) -> bool:
        return self.tpl.is_last_stage()

    def is_input_rank(self) -> bool:
        return self.tpl.is_first_stage()

    def is_output_rank(self) -> bool:
        return self.tpl.is_last_stage() and self.tpl.tp_rank == 0 and self.tpl.dp_rank == 0

    def get_rank(self) -> int:
        return self.comm.rank

    def get_local_rank(self) -> int:
        return self.comm.local_rank

    def get_world_size(self) -> int:
        return self.comm.world_size

    def barrier(self) -> None:
        """Host-side (gloo) barrier: safe when several ranks share one GPU under MPS."""
        self.comm.barrier()

    def apply_lora(self, cfg):
        return self._e.apply_lora(cfg)

    def load_lora_ckpt(self, step: int, epoch: int, lora_dir: Optional[str] = None):
        return self._e.load_lora_ckpt(step, epoch, lora_dir)

    def merge_lora(self):
        return self._e.merge_lora()

    @torch.no_grad()
    def forward(self, input_ids: Optional[torch.Tensor], attention_mask: Optional[torch.Tensor] = None):
        """One full forward; returns the model output on the last stage, else None."""
        if self._schedule_infer is None:
            self._schedule_infer = ScheduleInference(self)
        inputs = None
        if self.tpl.is_first_stage():
            inputs = {"input_ids": input_ids}
            if self.use_kv_cache:
                S = input_ids.shape[1]
                inputs["position_ids"] = torch.arange(S, device=input_ids.device).unsqueeze(0).expand(input_ids.shape[0], S)
        for ad in self._adaptors:
            ad.enabled = False
        try:
            return self._schedule_infer.run(inputs)
        finally:
            for ad in self._adaptors:
                ad.enabled = True

    __call__ = forward

    # ---- generation -------------------------------------------------------------------------------------
    def _next_token_exchange(self, token: Optional[torch.Tensor], done: bool, batch: int):
        """Last stage -> every stage of this pipeline: the sampled tokens and the stop flag, in one broadcast."""
        if self.tpl.pp_size == 1:
            return token, done
        buf = torch.zeros(batch + 1, dtype=torch.int64, device=self.device)
        if self.tpl.is_last_stage():
            buf[:batch] = token
            buf[batch] = int(done)
        dist.broadcast(buf, src=self.tpl.get_last_rank(), group=self.tpl.pp_group)
        return buf[:batch], bool(buf[batch].item())

    @torch.no_grad()
    def generate(self, input_ids: Optional[torch.Tensor] = None, max_new_tokens: int = 100, temperature: float = 1.0,
                 top_k: int = 50, top_p: float = 0.95, do_sample: bool = True, eos_token_id: Optional[int] = None,
                 pad_token_id: Optional[int] = None, streamer: Optional[Any] = None, verbose: bool = True) -> Optional[torch.Tensor]:
        first, last = self.tpl.is_first_stage(), self.tpl.is_last_stage()
        if first:
            if input_ids is None:
                raise ValueError("input_ids are required on the first stage")
            input_ids = self._to_device(input_ids)
        # the prompt is needed on the first stage (to run) and on the last (to assemble the result)
        if self.tpl.pp_size > 1:
            shape = torch.zeros(2, dtype=torch.int64, device=self.device)
            if first:
                shape[0], shape[1] = input_ids.shape
            dist.broadcast(shape, src=self.tpl.get_first_rank(), group=self.tpl.pp_group)
            B, S0 = int(shape[0]), int(shape[1])
            if not first:
                input_ids = torch.zeros(B, S0, dtype=torch.int64, device=self.device)
            dist.broadcast(input_ids, src=self.tpl.get_first_rank(), group=self.tpl.pp_group)
        else:
            B, S0 = input_ids.shape
        if S0 + max_new_tokens > self.max_seq_len and self.use_kv_cache:
            raise ValueError(f"prompt {S0} + max_new_tokens {max_new_tokens} exceeds max_seq_len {self.max_seq_len}")
        pad = pad_token_id if pad_token_id is not None else (eos_token_id if eos_token_id is not None else 0)
        out_ids = torch.full((B, S0 + max_new_tokens), pad, dtype=torch.int64, device=self.device)
        out_ids[:, :S0] = input_ids
        finished = torch.zeros(B, dtype=torch.bool, device=self.device)
        if streamer is not None and self.is_output_rank():
            streamer.put(input_ids.cpu())
        gen = None
        if self.use_kv_cache:
            if self._schedule_gen is None:
                self._schedule_gen = ScheduleGeneration(self)
            gen = self._schedule_gen
            self._ensure_cache(B)
            self.clear_kv_cache()
        elif self._schedule_infer is None:
            self._schedule_infer = ScheduleInference(self)
        cur = S0
        n_generated = 0
        token = None
        for step in range(max_new_tokens):
            if gen is not None:
                logits = gen.prefill(input_ids if first else None) if step == 0 else gen.decode_step(token if first else None, cur - 1)
            else:
                out = self._schedule_infer.run({"input_ids": out_ids[:, :cur]} if first else None)
                logits = None
                if last:
                    lg = out["logits"] if isinstance(out, dict) else (out[0] if isinstance(out, (tuple, list)) else out)
                    logits = lg[:, -1, :]
            done = False
            if last:
                token = sample_token(logits, temperature, top_k, top_p, do_sample)
                if eos_token_id is not None:
                    token = torch.where(finished, torch.full_like(token, pad), token)
                    finished = finished | (token == eos_token_id)
                    done = bool(finished.all().item())
            token, done = self._next_token_exchange(token, done, B)
            out_ids[:, cur] = token
            cur += 1
            n_generated += 1
            if streamer is not None and self.is_output_rank():
                streamer.put(token.cpu())
            if done:
                break
        if streamer is not None and self.is_output_rank():
            streamer.end()
        if self.use_kv_cache and not self.serving_mode:
            self.free_kv_cache()
        elif self.use_kv_cache:
            self.clear_kv_cache()
        return out_ids[:, :cur] if last else None
