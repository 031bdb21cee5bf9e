"""Fused Llama-family decoder layer for B200.

A traced HuggingFace Llama keeps each ``*DecoderLayer`` as one ``call_module``
node; the rewrite pass swaps it for :class:`B200LlamaLayer`, which computes the
same function with

* one packed QKV GEMM and one packed gate/up GEMM (tcgen05 kernel) instead of
  five projections,
* RoPE applied in place on the packed projection, causal flash attention
  reading q/k/v straight from it (no transposes, no ``repeat_kv``),
* residual-add fused into the RMSNorm kernel, SwiGLU fused,
* Megatron-style tensor parallelism (column split of QKV / gate-up, row split
  of out-proj / down-proj) with optional sequence parallelism: the residual
  stream is sharded along the sequence inside the TP group, an all-gather feeds
  the column GEMMs and a reduce-scatter follows the row GEMMs.

The reference shards the unfused HF modules with DTensor column/row plans and
has no sequence parallelism (opt_prime/opt_prime/opti_pri.py:887-1008).
Weights keep a mapping to HF names (:meth:`B200LlamaLayer.hf_state`) so
checkpoints stay HF-compatible.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import attention as attn_ops
from ..parallel import tp_comm

LEAF_CLASS_SUFFIX = "DecoderLayer"

__all__ = ["B200LlamaLayer", "FusedRMSNorm", "FusedLinear", "FusedEmbedding", "LEAF_CLASS_SUFFIX", "is_llama_layer"]


def is_llama_layer(m: nn.Module) -> bool:
    a, f = getattr(m, "self_attn", None), getattr(m, "mlp", None)
    return (a is not None and f is not None and all(hasattr(a, n) for n in ("q_proj", "k_proj", "v_proj", "o_proj"))
            and all(hasattr(f, n) for n in ("gate_proj", "up_proj", "down_proj"))
            and hasattr(m, "input_layernorm") and hasattr(m, "post_attention_layernorm"))


def _shard_rows(w: torch.Tensor, parts: int, idx: int) -> torch.Tensor:
    n = w.shape[0] // parts
    return w[idx * n:(idx + 1) * n]


def _shard_cols(w: torch.Tensor, parts: int, idx: int) -> torch.Tensor:
    n = w.shape[1] // parts
    return w[:, idx * n:(idx + 1) * n]


class B200LlamaLayer(nn.Module):
    def __init__(self, hf_layer: nn.Module, config, tp_size: int = 1, tp_rank: int = 0):
        super().__init__()
        attn, mlp = hf_layer.self_attn, hf_layer.mlp
        self.hidden = config.hidden_size
        self.n_heads = config.num_attention_heads
        self.n_kv = getattr(config, "num_key_value_heads", self.n_heads)
        self.head_dim = getattr(config, "head_dim", None) or self.hidden // self.n_heads
        self.inter = config.intermediate_size
        self.eps = float(getattr(config, "rms_norm_eps", 1e-6))
        self.theta = float(_rope_theta(config))
        self.rope_scaling = _rope_scaling(config)
        self.max_pos = int(getattr(config, "max_position_embeddings", 8192))
        self.layer_idx = getattr(attn, "layer_idx", 0)
        if self.n_heads % tp_size or self.n_kv % tp_size or self.inter % tp_size:
            raise ValueError(f"heads {self.n_heads}/{self.n_kv} and ffn {self.inter} must divide by tp_size {tp_size}")
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.tp_group = None
        self.sequence_parallel = False
        self.sp_first = self.sp_last = False
        self.tp_backend = "nccl"
        self.hq, self.hkv = self.n_heads // tp_size, self.n_kv // tp_size
        for lin in (attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj, mlp.gate_proj, mlp.up_proj, mlp.down_proj):
            if lin.bias is not None:
                raise ValueError("fused Llama layer expects bias-free projections")
        with torch.no_grad():
            qkv = torch.cat([_shard_rows(attn.q_proj.weight, tp_size, tp_rank), _shard_rows(attn.k_proj.weight, tp_size, tp_rank),
                             _shard_rows(attn.v_proj.weight, tp_size, tp_rank)], 0)
            gu = torch.cat([_shard_rows(mlp.gate_proj.weight, tp_size, tp_rank), _shard_rows(mlp.up_proj.weight, tp_size, tp_rank)], 0)
            o = _shard_cols(attn.o_proj.weight, tp_size, tp_rank)
            d = _shard_cols(mlp.down_proj.weight, tp_size, tp_rank)
            self.qkv_weight = nn.Parameter(qkv.detach().clone().contiguous())
            self.o_weight = nn.Parameter(o.detach().clone().contiguous())
            self.gate_up_weight = nn.Parameter(gu.detach().clone().contiguous())
            self.down_weight = nn.Parameter(d.detach().clone().contiguous())
            self.input_norm_weight = nn.Parameter(hf_layer.input_layernorm.weight.detach().clone())
            self.post_norm_weight = nn.Parameter(hf_layer.post_attention_layernorm.weight.detach().clone())
        for p in (self.qkv_weight, self.o_weight, self.gate_up_weight, self.down_weight):
            p.tp_sharded = True
        self._tables: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
        self.kv_cache = None  # set by the inference engine (paged or dense cache adaptor)
        self.lora = nn.ModuleDict()  # target name -> LoRAAdapter (empty unless apply_lora was called)
        self.lora_merged = False

    # ---- configuration by the engine -----------------------------------------
    def configure_tp(self, group, sequence_parallel: bool, sp_first: bool, sp_last: bool, backend: str = "nccl") -> None:
        self.tp_group = group
        self.sequence_parallel = sequence_parallel and self.tp_size > 1
        self.sp_first, self.sp_last = sp_first, sp_last
        self.tp_backend = backend
        for p in (self.input_norm_weight, self.post_norm_weight):
            p.sequence_parallel = self.sequence_parallel

    # ---- LoRA ---------------------------------------------------------------------------
    def _lora_dims(self):
        D, H, I = self.head_dim, self.hidden, self.inter // self.tp_size
        return {"q_proj": (H, self.hq * D), "k_proj": (H, self.hkv * D), "v_proj": (H, self.hkv * D),
                "o_proj": (self.hq * D, H), "gate_proj": (H, I), "up_proj": (H, I), "down_proj": (I, H)}

    def add_lora(self, cfg, tp_group=None, tp_size: int = 1) -> int:
        from ..lora import COLWISE_TARGETS, LoRAAdapter, _tp_grad_hook
        dims = self._lora_dims()
        w = self.qkv_weight
        n = 0
        for t in cfg.target_modules:
            if t not in dims or t in self.lora:
                continue
            fin, fout = dims[t]
            ad = LoRAAdapter(fin, fout, cfg.r, cfg.alpha, cfg.dropout, w.dtype, w.device)
            if tp_size > 1 and tp_group is not None:
                rep = ad.lora_A.weight if t in COLWISE_TARGETS else ad.lora_B.weight  # the replicated half
                dist_src = torch.distributed.get_global_rank(tp_group, 0)
                torch.distributed.broadcast(rep.data, src=dist_src, group=tp_group)
                rep.register_hook(_tp_grad_hook(tp_group, tp_size))
                (ad.lora_B.weight if t in COLWISE_TARGETS else ad.lora_A.weight).tp_sharded = True
            self.lora[t] = ad
            n += 1
        return n

    def _lora_cat(self, x, names):
        """Concatenated adapter outputs for the packed projection made of ``names`` (zeros where a target has no adapter)."""
        if not self.lora or self.lora_merged:
            return None
        dims = self._lora_dims()
        parts, any_ad = [], False
        for t in names:
            if t in self.lora:
                parts.append(self.lora[t](x))
                any_ad = True
            else:
                parts.append(x.new_zeros(*x.shape[:-1], dims[t][1]))
        return torch.cat(parts, -1) if any_ad else None

    def merge_lora(self) -> None:
        if not self.lora or self.lora_merged:
            return
        D = self.head_dim
        with torch.no_grad():
            offs = {"q_proj": 0, "k_proj": self.hq * D, "v_proj": (self.hq + self.hkv) * D}
            for t, o in offs.items():
                if t in self.lora:
                    dw = self.lora[t].delta_weight().to(self.qkv_weight.dtype)
                    self.qkv_weight.data[o:o + dw.shape[0]] += dw
            I = self.inter // self.tp_size
            for t, o in {"gate_proj": 0, "up_proj": I}.items():
                if t in self.lora:
                    self.gate_up_weight.data[o:o + I] += self.lora[t].delta_weight().to(self.gate_up_weight.dtype)
            if "o_proj" in self.lora:
                self.o_weight.data += self.lora["o_proj"].delta_weight().to(self.o_weight.dtype)
            if "down_proj" in self.lora:
                self.down_weight.data += self.lora["down_proj"].delta_weight().to(self.down_weight.dtype)
        self.lora_merged = True

    def _rope_tables(self, device) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._tables is None or self._tables[0].device != device:
            self._tables = ops.rope_tables(self.max_pos, self.head_dim, self.theta, device, self.rope_scaling)
        return self._tables

    # ---- forward -----------------------------------------------------------------
    def forward(self, hidden_states: torch.Tensor, attention_mask=None, position_ids: Optional[torch.Tensor] = None,
                past_key_values=None, use_cache=False, position_embeddings=None, **kwargs) -> torch.Tensor:
        sp = self.sequence_parallel
        tp = self.tp_size > 1
        if sp and self.sp_first:
            hidden_states = tp_comm.scatter_to_sp(hidden_states, self.tp_group, self.tp_rank, self.tp_size)
        B, S_loc, H = hidden_states.shape
        S = S_loc * self.tp_size if sp else S_loc
        residual = hidden_states
        x, _ = ops.rmsnorm(hidden_states, self.input_norm_weight, self.eps)
        # --- attention block
        use_lora = bool(self.lora) and not self.lora_merged
        if sp and not use_lora:
            qkv = tp_comm.allgather_linear(x, self.qkv_weight, self.tp_group, self.tp_size, self.tp_backend)
        else:
            if sp:
                x = tp_comm.gather_seq(x, self.tp_group, self.tp_size)
            elif tp:
                x = tp_comm.copy_to_tp(x, self.tp_group)
            qkv = ops.linear(x, self.qkv_weight)
            if use_lora:
                dl = self._lora_cat(x, ("q_proj", "k_proj", "v_proj"))
                if dl is not None:
                    qkv = qkv + dl
        qkv = qkv.reshape(B * S, (self.hq + 2 * self.hkv) * self.head_dim)
        if position_ids is None:
            pos = torch.arange(S, device=qkv.device, dtype=torch.int32).repeat(B)
        else:
            pos = position_ids.expand(B, S).reshape(-1).to(torch.int32)
        cos, sin = self._rope_tables(qkv.device)
        if self.max_pos < S:
            raise ValueError(f"sequence of {S} exceeds max_position_embeddings {self.max_pos}")
        qkv = ops.apply_rope_qkv(qkv, pos, cos, sin, self.hq + self.hkv, self.head_dim)
        if self.kv_cache is not None:
            a = self.kv_cache.attend(self, qkv, B, S, pos)
        else:
            a = attn_ops.causal_attention_packed(qkv, B, S, self.hq, self.hkv, self.head_dim)
        a = a.view(B, S, -1)
        if sp and not (use_lora and "o_proj" in self.lora):
            o = tp_comm.linear_reducescatter(a, self.o_weight, self.tp_group, self.tp_size, self.tp_backend)
        else:
            o = ops.linear(a, self.o_weight)
            if use_lora and "o_proj" in self.lora:
                o = o + self.lora["o_proj"](a)
            if sp:
                o = tp_comm.reduce_scatter_seq(o, self.tp_group, self.tp_size)
            elif tp:
                o = tp_comm.reduce_from_tp(o, self.tp_group)
        # --- MLP block (residual add fused into the norm)
        x, residual = ops.rmsnorm(o, self.post_norm_weight, self.eps, residual=residual)
        if sp and not use_lora:
            gu = tp_comm.allgather_linear(x, self.gate_up_weight, self.tp_group, self.tp_size, self.tp_backend)
        else:
            if sp:
                x = tp_comm.gather_seq(x, self.tp_group, self.tp_size)
            elif tp:
                x = tp_comm.copy_to_tp(x, self.tp_group)
            gu = ops.linear(x, self.gate_up_weight)
            if use_lora:
                dl = self._lora_cat(x, ("gate_proj", "up_proj"))
                if dl is not None:
                    gu = gu + dl
        act = ops.swiglu(gu)
        if sp and not (use_lora and "down_proj" in self.lora):
            d = tp_comm.linear_reducescatter(act, self.down_weight, self.tp_group, self.tp_size, self.tp_backend)
        else:
            d = ops.linear(act, self.down_weight)
            if use_lora and "down_proj" in self.lora:
                d = d + self.lora["down_proj"](act)
            if sp:
                d = tp_comm.reduce_scatter_seq(d, self.tp_group, self.tp_size)
            elif tp:
                d = tp_comm.reduce_from_tp(d, self.tp_group)
        out = residual + d
        if sp and self.sp_last:
            out = tp_comm.gather_from_sp(out, self.tp_group, self.tp_rank, self.tp_size)
        return out

    # ---- HF-compatible view of the weights -------------------------------------------
    def hf_state(self, prefix: str) -> Dict[str, torch.Tensor]:
        """This rank's shard under HF parameter names (q/k/v/gate/up are row shards, o/down column shards)."""
        D = self.head_dim
        q, k, v = torch.split(self.qkv_weight.detach(), [self.hq * D, self.hkv * D, self.hkv * D], 0)
        g, u = torch.split(self.gate_up_weight.detach(), [self.inter // self.tp_size] * 2, 0)
        return {
            f"{prefix}self_attn.q_proj.weight": q, f"{prefix}self_attn.k_proj.weight": k, f"{prefix}self_attn.v_proj.weight": v,
            f"{prefix}self_attn.o_proj.weight": self.o_weight.detach(),
            f"{prefix}mlp.gate_proj.weight": g, f"{prefix}mlp.up_proj.weight": u, f"{prefix}mlp.down_proj.weight": self.down_weight.detach(),
            f"{prefix}input_layernorm.weight": self.input_norm_weight.detach(),
            f"{prefix}post_attention_layernorm.weight": self.post_norm_weight.detach(),
        }

    def load_hf_state(self, prefix: str, sd: Dict[str, torch.Tensor]) -> None:
        """Inverse of :meth:`hf_state` for full (unsharded) HF tensors."""
        t, r = self.tp_size, self.tp_rank
        with torch.no_grad():
            q = _shard_rows(sd[f"{prefix}self_attn.q_proj.weight"], t, r)
            k = _shard_rows(sd[f"{prefix}self_attn.k_proj.weight"], t, r)
            v = _shard_rows(sd[f"{prefix}self_attn.v_proj.weight"], t, r)
            self.qkv_weight.copy_(torch.cat([q, k, v], 0))
            g = _shard_rows(sd[f"{prefix}mlp.gate_proj.weight"], t, r)
            u = _shard_rows(sd[f"{prefix}mlp.up_proj.weight"], t, r)
            self.gate_up_weight.copy_(torch.cat([g, u], 0))
            self.o_weight.copy_(_shard_cols(sd[f"{prefix}self_attn.o_proj.weight"], t, r))
            self.down_weight.copy_(_shard_cols(sd[f"{prefix}mlp.down_proj.weight"], t, r))
            self.input_norm_weight.copy_(sd[f"{prefix}input_layernorm.weight"])
            self.post_norm_weight.copy_(sd[f"{prefix}post_attention_layernorm.weight"])


def _rope_theta(config) -> float:
    rp = getattr(config, "rope_parameters", None)
    if isinstance(rp, dict) and "rope_theta" in rp:
        return rp["rope_theta"]
    return getattr(config, "rope_theta", 10000.0)


def _rope_scaling(config) -> Optional[dict]:
    rp = getattr(config, "rope_parameters", None)
    if isinstance(rp, dict) and rp.get("rope_type", "default") not in ("default", None):
        return rp
    rs = getattr(config, "rope_scaling", None)
    if isinstance(rs, dict) and rs.get("rope_type", rs.get("type", "default")) not in ("default", None):
        return rs
    return None


# ---------------------------------------------------------------------- per-op substitutes (generic path)
class FusedRMSNorm(nn.Module):
    def __init__(self, hf_norm: nn.Module):
        super().__init__()
        self.weight = hf_norm.weight
        self.eps = float(getattr(hf_norm, "variance_epsilon", getattr(hf_norm, "eps", 1e-6)))

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)[0]


class FusedLayerNorm(nn.Module):
    def __init__(self, ln: nn.LayerNorm):
        super().__init__()
        self.weight, self.bias, self.eps = ln.weight, ln.bias, ln.eps

    def forward(self, x):
        return ops.layernorm(x, self.weight, self.bias, self.eps)[0]


class FusedLinear(nn.Module):
    def __init__(self, lin: nn.Linear):
        super().__init__()
        self.weight, self.bias = lin.weight, lin.bias
        self.in_features, self.out_features = lin.in_features, lin.out_features

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class FusedConv1D(nn.Module):
    """HF ``Conv1D`` (GPT-2 family): a linear layer whose weight is stored ``[in, out]``; same parameters, tcgen05 GEMMs."""

    def __init__(self, conv):
        super().__init__()
        self.weight, self.bias = conv.weight, conv.bias
        self.nf = conv.nf

    def forward(self, x):
        return ops.linear_kn(x, self.weight, self.bias)


class FusedEmbedding(nn.Module):
    def __init__(self, emb: nn.Embedding):
        super().__init__()
        self.weight = emb.weight
        self.num_embeddings, self.embedding_dim = emb.num_embeddings, emb.embedding_dim

    def forward(self, ids):
        return ops.embedding(ids, self.weight)
