"""Kernel substitution pass over a traced module-level graph.

Swaps library-backed modules for implementations built on this framework's
sm_100a kernels, in place on the ``GraphModule``:

* Llama-family ``*DecoderLayer`` leaves -> :class:`~aicomp_b200.models.llama.B200LlamaLayer`
  (fused QKV / gate-up GEMMs, in-place RoPE, flash attention, fused add+RMSNorm,
  tensor/sequence-parallel aware).  Keyword arguments the fused layer does not
  need (masks, caches, precomputed rotary tuples) are dropped from the call, so
  their producers disappear from the graph and are not relayed between stages.
* ``*RMSNorm`` -> fused RMSNorm, ``nn.LayerNorm`` -> fused LayerNorm,
  ``nn.Linear`` -> tcgen05 GEMM linear, ``nn.Embedding`` -> gather kernel.

Every substitute has a PyTorch path for CPU / fp32 tensors, so a rewritten
graph runs (and is tested) without a GPU.
"""
from __future__ import annotations

from typing import Dict

import torch.fx as fx
import torch.nn as nn

from ..models import llama as _llama

_DROP_KWARGS = ("attention_mask", "past_key_values", "past_key_value", "use_cache", "position_embeddings", "cache_position",
                "output_attentions")


def _set_submodule(root: nn.Module, path: str, new: nn.Module) -> None:
    parent_path, _, name = path.rpartition(".")
    parent = root.get_submodule(parent_path) if parent_path else root
    setattr(parent, name, new)


def substitute_kernels(gm: fx.GraphModule, model: nn.Module, tp_size: int = 1, tp_rank: int = 0) -> Dict[str, int]:
    """Rewrite ``gm`` in place; returns ``{kind: count}`` of substitutions."""
    import os
    tp_rank = int(os.environ.get("RANK", "0")) % tp_size if tp_size > 1 else 0
    config = getattr(model, "config", None)
    counts: Dict[str, int] = {}
    layer_nodes = []
    for node in list(gm.graph.nodes):
        if node.op != "call_module":
            continue
        target = str(node.target)
        mod = gm.get_submodule(target)
        cname = type(mod).__name__
        new = None
        if cname.endswith(_llama.LEAF_CLASS_SUFFIX) and _llama.is_llama_layer(mod) and config is not None:
            new = _llama.B200LlamaLayer(mod, config, tp_size=tp_size, tp_rank=tp_rank)
            node.kwargs = {k: v for k, v in node.kwargs.items() if k not in _DROP_KWARGS}
            layer_nodes.append(node)
            kind = "llama_layer"
        elif cname.endswith("RMSNorm") and hasattr(mod, "weight"):
            new, kind = _llama.FusedRMSNorm(mod), "rmsnorm"
        elif type(mod) is nn.LayerNorm and mod.elementwise_affine:
            new, kind = _llama.FusedLayerNorm(mod), "layernorm"
        elif type(mod) is nn.Linear:
            new, kind = _llama.FusedLinear(mod), "linear"
        elif cname == "Conv1D" and hasattr(mod, "nf") and getattr(mod, "weight", None) is not None and mod.weight.dim() == 2:
            new, kind = _llama.FusedConv1D(mod), "conv1d"
        elif type(mod) is nn.Embedding and mod.padding_idx is None and mod.max_norm is None:
            new, kind = _llama.FusedEmbedding(mod), "embedding"
        if new is not None:
            _set_submodule(gm, target, new)
            counts[kind] = counts.get(kind, 0) + 1
    if layer_nodes:
        layer_nodes[0].meta["sp_first"] = True
        layer_nodes[-1].meta["sp_last"] = True
        gm.get_submodule(str(layer_nodes[0].target))._sp_first_in_model = True
        gm.get_submodule(str(layer_nodes[-1].target))._sp_last_in_model = True
    gm.graph.eliminate_dead_code()
    gm.recompile()
    return counts
