"""HF-compatible distributed checkpoint: one ``stage{S}_tp{T}.pt`` per (stage, tp rank).

Format of the reference (opt_prime/opt_prime/opti_pri.py:1026-1088): a dict with keys ``stage, tp_rank,
tp_size, pp_size, step, epoch, state_dict``; only data-parallel replica 0 writes; LoRA adapter tensors are
left out and ``.base_linear.`` is unwrapped.  Stage modules here keep real HF parameter names, and the fused
Llama layers export their packed weights under the separate HF projection names, so
:mod:`aicomp_b200.ckpt.merge_hf_ckpt` (and the reference's merge tool) can rebuild a standard HF model.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch
import torch.nn as nn


def stage_hf_state_dict(stage_module: nn.Module) -> Dict[str, torch.Tensor]:
    """State dict of a stage under HF names (this rank's TP shard for sharded projections)."""
    from ..models.llama import B200LlamaLayer
    fused_prefixes = {}
    for name, m in stage_module.named_modules():
        if isinstance(m, B200LlamaLayer):
            fused_prefixes[name + "."] = m
    out: Dict[str, torch.Tensor] = {}
    for key, val in stage_module.state_dict().items():
        if any(key.startswith(p) for p in fused_prefixes):
            continue
        if "lora_A" in key or "lora_B" in key:
            continue
        key = key.replace(".base_linear.", ".")
        out[key] = val.detach().cpu()
    for prefix, m in fused_prefixes.items():
        for k, v in m.hf_state(prefix).items():
            out[k] = v.detach().cpu().contiguous()
    return out


def save_hf_ckpt(engine, save_dir: str, step: Optional[int] = None, epoch: Optional[int] = None) -> Optional[str]:
    if engine.use_gpu:
        torch.cuda.synchronize()
    if engine.tpl.dp_rank != 0:
        return None
    sd = stage_hf_state_dict(engine.stage_module)
    os.makedirs(save_dir, exist_ok=True)
    stage, tp_rank = engine.tpl.stage, engine.tpl.tp_rank
    path = os.path.join(save_dir, f"stage{stage}_tp{tp_rank}.pt")
    tmp = path + ".tmp"
    torch.save({"stage": stage, "tp_rank": tp_rank, "tp_size": engine.tpl.tp_size, "pp_size": engine.tpl.pp_size,
                "step": step, "epoch": epoch, "state_dict": sd}, tmp)
    os.replace(tmp, path)
    return path
