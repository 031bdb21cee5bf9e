"""Give a stage module real storage on its device.

Models may arrive on the ``meta`` device (nothing allocated): only the stage a
rank owns is materialised, straight on its GPU, and initialised there.  Models
with real weights are moved (and optionally cast).  Sized for 180 GB HBM3e: a
Llama-3-8B stage never exists in host memory.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn


def default_init_(module: nn.Module, std: float = 0.02) -> None:
    """N(0, std) for weights of linear/embedding-like modules, ones for norm weights, zeros for biases."""
    for m in module.modules():
        own = dict(m.named_parameters(recurse=False))
        if not own:
            continue
        cname = type(m).__name__.lower()
        for name, p in own.items():
            with torch.no_grad():
                if "norm" in cname or name.endswith("norm_weight"):
                    (p.zero_() if "bias" in name else p.fill_(1.0))
                elif "bias" in name:
                    p.zero_()
                else:
                    p.normal_(0.0, std)


def _reinit_buffers(module: nn.Module, device) -> None:
    for m in module.modules():
        # HF rotary embeddings keep inv_freq as a computed, non-persistent buffer
        if hasattr(m, "rope_init_fn") and hasattr(m, "config") and hasattr(m, "inv_freq"):
            try:
                inv_freq, scaling = m.rope_init_fn(m.config, device)
                m.register_buffer("inv_freq", inv_freq, persistent=False)
                if hasattr(m, "original_inv_freq"):
                    m.register_buffer("original_inv_freq", inv_freq.clone(), persistent=False)
                m.attention_scaling = scaling
            except Exception:
                pass
        if hasattr(m, "reset_buffers"):
            m.reset_buffers(device)


def materialize_module(module: nn.Module, device: torch.device, dtype: Optional[torch.dtype] = None,
                       init_fn: Optional[Callable[[nn.Module], None]] = None, root: Optional[nn.Module] = None) -> nn.Module:
    has_meta = any(p.is_meta for p in module.parameters()) or any(b.is_meta for b in module.buffers())
    if has_meta:
        real = {n: p for n, p in module.named_parameters() if not p.is_meta}
        if real:
            raise ValueError("a model must be entirely on the meta device or entirely materialised")
        module.to_empty(device=device)
        if dtype is not None:
            for p in module.parameters():
                if p.is_floating_point():
                    p.data = p.data.to(dtype)
        std = 0.02
        cfg = getattr(root, "config", None)
        if cfg is not None and hasattr(cfg, "initializer_range"):
            std = float(cfg.initializer_range)
        (init_fn or (lambda m: default_init_(m, std)))(module)
        _reinit_buffers(module, device)
    else:
        module.to(device)
        if dtype is not None:
            for p in module.parameters():
                if p.is_floating_point() and p.dtype != dtype:
                    p.data = p.data.to(dtype)
            for b in module.buffers():
                if b.is_floating_point() and b.dtype not in (torch.float32,) and b.dtype != dtype:
                    b.data = b.data.to(dtype)
    return module
