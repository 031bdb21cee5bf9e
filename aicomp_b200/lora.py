"""LoRA fine-tuning on top of the pipeline / tensor-parallel engine.

Same user surface as the reference (opt_prime/opt_prime/lora.py:24-314 and the engine glue at
opti_pri.py:1092-1190): ``LoRAConfig(r, alpha, dropout, target_modules)``, ``apply_lora`` freezes the base
weights and trains only ``lora_A`` (Kaiming) / ``lora_B`` (zeros) with ``scaling = alpha / r``;
``merge_lora`` folds the adapters into the base weights; adapters are saved per stage as
``lora_checkpoint_stage_<s>/lora_step_<s>_epoch_<e>[_tp<r>].pt``.

Two hosts for adapters: :class:`LoRALinear` wraps ordinary linear modules of a traced graph; fused Llama
layers keep their packed QKV / gate-up GEMMs and add the low-rank terms per target on the matching
column slices.  Under tensor parallelism the half of each adapter that follows the base weight's split is
sharded (``lora_B`` for column-split targets, ``lora_A`` for row-split ones); the other half is replicated
and its gradient is averaged over the TP group by a hook, as in the reference (lora.py:206-262).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

__all__ = ["LoRAConfig", "LoRALinear", "LoRAAdapter", "apply_lora_to_module", "lora_state_dict", "load_lora_state_dict"]

COLWISE_TARGETS = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
ROWWISE_TARGETS = ("o_proj", "down_proj")


@dataclass
class LoRAConfig:
    r: int = 8
    alpha: float = 16.0
    dropout: float = 0.05
    target_modules: List[str] = field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"])


class LoRAAdapter(nn.Module):
    """``delta(x) = scaling * B(A(dropout(x)))`` with ``A: in -> r`` and ``B: r -> out``."""

    def __init__(self, in_features: int, out_features: int, r: int, alpha: float, dropout: float, dtype, device):
        super().__init__()
        self.lora_A = nn.Linear(in_features, r, bias=False, dtype=dtype, device=device)
        self.lora_B = nn.Linear(r, out_features, bias=False, dtype=dtype, device=device)
        nn.init.kaiming_uniform_(self.lora_A.weight, a=math.sqrt(5))
        nn.init.zeros_(self.lora_B.weight)
        self.scaling = alpha / r
        self.drop = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    def forward(self, x):
        return self.lora_B(self.lora_A(self.drop(x))) * self.scaling

    def delta_weight(self) -> torch.Tensor:
        return (self.lora_B.weight @ self.lora_A.weight) * self.scaling


class LoRALinear(nn.Module):
    """Drop-in for a linear module: frozen base plus a trainable low-rank branch."""

    def __init__(self, base_linear: nn.Module, r: int, alpha: float, dropout: float = 0.0):
        super().__init__()
        self.base_linear = base_linear
        w = base_linear.weight
        self.adapter_in, self.adapter_out = w.shape[1], w.shape[0]
        ad = LoRAAdapter(w.shape[1], w.shape[0], r, alpha, dropout, w.dtype, w.device)
        self.lora_A, self.lora_B, self.lora_dropout = ad.lora_A, ad.lora_B, ad.drop
        self.r, self.scaling, self.merged = r, alpha / r, False
        for p in self.base_linear.parameters():
            p.requires_grad = False

    def forward(self, x):
        out = self.base_linear(x)
        if self.merged:
            return out
        return out + self.lora_B(self.lora_A(self.lora_dropout(x))) * self.scaling

    def merge_weights(self) -> None:
        if self.merged:
            return
        with torch.no_grad():
            w = self.base_linear.weight
            w.data += ((self.lora_B.weight.float() @ self.lora_A.weight.float()) * self.scaling).to(w.dtype)
        self.merged = True


def _tp_grad_hook(group, size):
    def hook(g):
        # every rank contributes the part of the gradient that flows through its shard of the other half:
        # the true gradient is the SUM (the reference divides by tp, lora.py:252-258, which scales it down)
        g = g.contiguous()
        dist.all_reduce(g, group=group)
        return g
    return hook


def apply_lora_to_module(stage_module: nn.Module, cfg: LoRAConfig, tp_group=None, tp_size: int = 1) -> int:
    """Freeze everything, then add adapters to every target; returns the number of adapted projections."""
    from .models.llama import B200LlamaLayer
    for p in stage_module.parameters():
        p.requires_grad = False
    n = 0
    for name, m in list(stage_module.named_modules()):
        if isinstance(m, B200LlamaLayer):
            n += m.add_lora(cfg, tp_group, tp_size)
    for name, m in list(stage_module.named_modules()):
        leaf = name.rsplit(".", 1)[-1]
        if leaf in cfg.target_modules and hasattr(m, "weight") and isinstance(getattr(m, "weight"), torch.Tensor) \
                and m.weight.dim() == 2 and not isinstance(m, LoRALinear) and not name.endswith("base_linear"):
            parent_name, _, attr = name.rpartition(".")
            parent = stage_module.get_submodule(parent_name) if parent_name else stage_module
            setattr(parent, attr, LoRALinear(m, cfg.r, cfg.alpha, cfg.dropout))
            n += 1
    return n


def lora_state_dict(stage_module: nn.Module) -> Dict[str, torch.Tensor]:
    return {k: v.detach().cpu() for k, v in stage_module.state_dict().items() if "lora_A" in k or "lora_B" in k}


def load_lora_state_dict(stage_module: nn.Module, sd: Dict[str, torch.Tensor]) -> None:
    own = stage_module.state_dict()
    missing = [k for k in sd if k not in own]
    if missing:
        raise KeyError(f"adapter keys not present in this stage: {missing[:4]}...")
    with torch.no_grad():
        for k, v in sd.items():
            own[k].copy_(v)


def merge_lora_in_module(stage_module: nn.Module) -> None:
    from .models.llama import B200LlamaLayer
    for m in stage_module.modules():
        if isinstance(m, LoRALinear):
            m.merge_weights()
        elif isinstance(m, B200LlamaLayer):
            m.merge_lora()


# ---- engine glue -------------------------------------------------------------------------------
def engine_apply_lora(engine, cfg: LoRAConfig) -> int:
    n = apply_lora_to_module(engine.stage_module, cfg, engine.tpl.tp_group, engine.tpl.tp_size)
    engine.lora_applied, engine.lora_config = True, cfg
    if getattr(engine, "dp", None) is not None:
        engine.dp.params = [p for p in engine.stage_module.parameters() if p.requires_grad]
        engine.dp.broadcast_parameters(src=engine.tpl.dp_ranks()[0])
    return n


def _lora_dir(engine, lora_dir: Optional[str]) -> str:
    return f"{lora_dir}_stage_{engine.tpl.stage}" if lora_dir else f"lora_checkpoint_stage_{engine.tpl.stage}"


def _lora_file(engine, step: int, epoch: int) -> str:
    suffix = f"_tp{engine.tpl.tp_rank}" if engine.tpl.tp_size > 1 else ""
    return f"lora_step_{step}_epoch_{epoch}{suffix}.pt"


def engine_save_lora(engine, step: int, epoch: int, lora_dir: Optional[str] = None) -> Optional[str]:
    if not engine.lora_applied:
        raise RuntimeError("apply_lora() first")
    if engine.tpl.dp_rank != 0:
        return None
    d = _lora_dir(engine, lora_dir)
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, _lora_file(engine, step, epoch))
    cfg = engine.lora_config
    torch.save({"step": step, "epoch": epoch, "stage": engine.tpl.stage, "tp_rank": engine.tpl.tp_rank,
                "lora_config": {"r": cfg.r, "alpha": cfg.alpha, "dropout": cfg.dropout, "target_modules": list(cfg.target_modules)},
                "lora_state_dict": lora_state_dict(engine.stage_module)}, path + ".tmp")
    os.replace(path + ".tmp", path)
    return path


def engine_load_lora(engine, step: int, epoch: int, lora_dir: Optional[str] = None) -> None:
    if not engine.lora_applied:
        raise RuntimeError("apply_lora() first")
    path = os.path.join(_lora_dir(engine, lora_dir), _lora_file(engine, step, epoch))
    blob = torch.load(path, map_location="cpu", weights_only=False)
    load_lora_state_dict(engine.stage_module, blob["lora_state_dict"])


def engine_merge_lora(engine) -> None:
    merge_lora_in_module(engine.stage_module)
