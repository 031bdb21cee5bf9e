"""Tensor-parallel set-up of a stage module.

The fused Llama layers are built already sharded (the rewrite pass slices the
projection weights for this rank); this module wires the process group into
them, turns sequence parallelism on, and finishes gradients of parameters that
are replicated across the group but see sharded activations.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.llama import B200LlamaLayer


def is_tp_duplicate(p: nn.Parameter) -> bool:
    """Parameters that every tensor-parallel rank holds in full (norm weights, embeddings, lm_head)."""
    return not getattr(p, "tp_sharded", False)


def apply_tensor_parallel(stage_module: nn.Module, tpl, sequence_parallel: bool = True, backend: str = "fused") -> None:
    layers: List[B200LlamaLayer] = [m for m in stage_module.modules() if isinstance(m, B200LlamaLayer)]
    if not layers:
        raise ValueError("tensor parallelism needs the fused Llama layers (fused_kernels=True)")
    for m in layers:
        m.configure_tp(tpl.tp_group, sequence_parallel, sp_first=getattr(m, "_sp_first_in_model", False),
                       sp_last=getattr(m, "_sp_last_in_model", False), backend=backend)
    # replicated parameters start identical on all TP ranks
    if tpl.tp_group is not None:
        src = tpl.tp_ranks()[0]
        for p in stage_module.parameters():
            if is_tp_duplicate(p):
                dist.broadcast(p.data, src=src, group=tpl.tp_group)


def finish_sequence_parallel_grads(stage_module: nn.Module, tpl) -> None:
    """Sum the gradients of replicated parameters that were computed from sequence shards (norm weights)."""
    if tpl.tp_group is None:
        return
    for p in stage_module.parameters():
        if getattr(p, "sequence_parallel", False):
            g = p.grad if p.grad is not None else getattr(p, "main_grad", None)
            if g is not None:
                dist.all_reduce(g, group=tpl.tp_group)
