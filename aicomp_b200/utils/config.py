"""Typed configuration on top of the keyword-argument API (YAML / JSON / command line).

The reference configures engines with constructor keywords only and ad-hoc ``argparse`` in every example
(opt_prime/opt_prime/opti_pri.py:350; examples/pp_inference_llama.py:95-200); its gpt-neox fork has a YAML->dataclass
system (gpt-neox/megatron/neox_arguments/arguments.py).  These dataclasses hold the same knobs, validate them, load
from files, and turn into the keyword dictionaries the engines take.
"""
from __future__ import annotations

import argparse
import json
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Dict, List, Optional


@dataclass
class ParallelConfig:
    pp_size: int = 1
    dp_size: int = 1
    tp_size: int = 1
    num_mb: int = 1
    sequence_parallel: bool = True
    partitioner: str = "auto"
    ir_analyze: str = "PARALLEL"
    dp_backend: str = "fused"
    tp_backend: str = "fused"

    def validate(self, world_size: Optional[int] = None) -> None:
        from ..graph.partition import PARTITIONERS
        if min(self.pp_size, self.dp_size, self.tp_size, self.num_mb) < 1:
            raise ValueError("parallel sizes and num_mb must be >= 1")
        if self.partitioner not in PARTITIONERS:
            raise ValueError(f"partitioner must be one of {PARTITIONERS}")
        if self.ir_analyze not in ("SINGLE", "PARALLEL", "SEQUENTIAL"):
            raise ValueError("ir_analyze must be SINGLE, PARALLEL or SEQUENTIAL")
        for b in (self.dp_backend, self.tp_backend):
            if b not in ("fused", "nccl"):
                raise ValueError("backends are 'fused' or 'nccl'")
        if world_size is not None and self.pp_size * self.dp_size * self.tp_size != world_size:
            raise ValueError(f"pp x dp x tp = {self.pp_size * self.dp_size * self.tp_size} != world size {world_size}")


@dataclass
class TrainConfig:
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    dtype: str = "bfloat16"
    schedule: str = "1f1b"
    activation_ckpt: bool = False
    lr: float = 1e-4
    betas: List[float] = field(default_factory=lambda: [0.9, 0.95])
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    checkpoint: bool = False
    ckpt_dir_postfix: Optional[str] = None
    use_padding: bool = True
    swap_opt_in_fwdbwd: bool = False
    swap_model_in_optstep: bool = False
    swap_use_disk: bool = False

    def engine_kwargs(self) -> Dict[str, Any]:
        import torch
        from ..engine import IR_Anal
        p = self.parallel
        return dict(num_mb=p.num_mb, pp_size=p.pp_size, dp_size=p.dp_size, tp_size=p.tp_size, partitioner=p.partitioner,
                    ir_analyze=IR_Anal[p.ir_analyze], sequence_parallel=p.sequence_parallel, dp_backend=p.dp_backend,
                    tp_backend=p.tp_backend, dtype=getattr(torch, self.dtype), activation_ckpt=self.activation_ckpt,
                    checkpoint=self.checkpoint, ckpt_dir_postfix=self.ckpt_dir_postfix, use_padding=self.use_padding,
                    swap_opt_in_fwdbwd=self.swap_opt_in_fwdbwd, swap_model_in_optstep=self.swap_model_in_optstep,
                    swap_use_disk=self.swap_use_disk)

    def optimizer_kwargs(self) -> Dict[str, Any]:
        return dict(lr=self.lr, betas=tuple(self.betas), weight_decay=self.weight_decay, max_grad_norm=self.max_grad_norm,
                    grad_scale=1.0 / self.parallel.num_mb)


@dataclass
class ServeConfig:
    tp_size: int = 1
    max_seqs: int = 256
    max_seq_len: int = 4096
    kv_block: int = 16
    kv_memory_fraction: float = 0.85
    cuda_graphs: bool = True
    max_prefill_per_step: int = 4
    disaggregated: bool = False
    prefill_gpus: int = 0
    decode_gpus: int = 0


def _from_dict(cls, d: Dict[str, Any]):
    known = {f.name: f for f in fields(cls)}
    unknown = set(d) - set(known)
    if unknown:
        raise ValueError(f"unknown {cls.__name__} keys: {sorted(unknown)}")
    kw = {}
    for k, v in d.items():
        if k == "parallel" and isinstance(v, dict):
            v = _from_dict(ParallelConfig, v)
        kw[k] = v
    return cls(**kw)


def load_config(path: str, cls=TrainConfig):
    """Load a YAML (``.yml`` / ``.yaml``) or JSON file into ``cls``; unknown keys are an error."""
    with open(path) as f:
        if path.endswith((".yml", ".yaml")):
            import yaml
            d = yaml.safe_load(f) or {}
        else:
            d = json.load(f)
    cfg = _from_dict(cls, d)
    if hasattr(cfg, "parallel"):
        cfg.parallel.validate()
    return cfg


def add_cli_arguments(ap: argparse.ArgumentParser, cls=ParallelConfig, prefix: str = "") -> None:
    for f in fields(cls):
        if f.type in ("int", "float", "str", "bool", int, float, str, bool):
            name = "--" + prefix + f.name.replace("_", "-")
            if f.type in ("bool", bool):
                ap.add_argument(name, type=lambda s: s.lower() in ("1", "true", "yes"), default=f.default)
            else:
                ap.add_argument(name, type={"int": int, "float": float, "str": str}.get(f.type, f.type), default=f.default)


def to_dict(cfg) -> Dict[str, Any]:
    return asdict(cfg)
