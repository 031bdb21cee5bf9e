"""``IR``: graph capture, partitioning and per-stage module set-up behind one object.

Method names mirror the reference's ``IR`` class (opt_prime/opt_prime/IR.py:1372-3015:
``retrieve_IR``, ``split_IR``, ``setup_submod``, ``cross_reference_analyze``,
``clean_module_memory``) so code written against it finds the same entry points.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.fx as fx
import torch.nn as nn

from ..utils.log import get_logger
from . import partition as _partition
from .split import StagePlan, build_stage_plan, extract_stage
from .tracer import trace_model

log = get_logger(__name__)

__all__ = ["IR"]


class IR:
    def __init__(self, module: nn.Module, engine=None):
        self.module = module
        self.engine = engine
        self.gm: Optional[fx.GraphModule] = None
        self.model_type = None
        self.input_names: List[str] = []
        self.assignment: Dict[fx.Node, int] = {}
        self.plan: Optional[StagePlan] = None
        self.special_nodes: Dict[str, Tuple[int, int]] = {}
        self.metadata_range: List[Tuple[int, str]] = []

    # ---- capture ------------------------------------------------------------
    def retrieve_IR(self, dynamo_capture: bool = False, example_inputs: Optional[Dict[str, Any]] = None,
                    input_names: Optional[List[str]] = None, use_kv_cache: bool = False, for_training: bool = True,
                    const_kwargs: Optional[Dict[str, Any]] = None) -> fx.GraphModule:
        e = self.engine
        fused = bool(getattr(e, "fused_kernels", False))
        leaf_classes: Tuple[str, ...] = ()
        if fused and getattr(e, "is_llama", False):
            from ..models.llama import LEAF_CLASS_SUFFIX
            leaf_classes = tuple({type(m).__name__ for m in self.module.modules() if type(m).__name__.endswith(LEAF_CLASS_SUFFIX)})
        if input_names is None and not for_training and use_kv_cache:
            input_names = ["input_ids", "position_ids"]  # generation feeds explicit positions (reference IR.py:1417-1419)
        if dynamo_capture:
            from .export_capture import export_to_module_graph
            res = export_to_module_graph(self.module, input_names=input_names, example_inputs=example_inputs, leaf_classes=leaf_classes)
        else:
            res = trace_model(self.module, input_names=input_names, example_inputs=example_inputs, leaf_classes=leaf_classes,
                              const_kwargs=const_kwargs)
        self.gm, self.input_names, self.model_type = res.gm, res.input_names, res.model_type
        if fused:
            from .rewrite import substitute_kernels
            substitute_kernels(self.gm, self.module, tp_size=getattr(getattr(e, "tpl", None), "tp_size", 1))
        return self.gm

    # ---- partition ------------------------------------------------------------
    def split_IR(self, method: str, num_stage: int) -> Dict[str, int]:
        e = self.engine
        asg = _partition.assign_stages(self.gm, num_stage, method, is_llama=bool(getattr(e, "is_llama", False)),
                                       tp_size=getattr(getattr(e, "tpl", None), "tp_size", 1))
        table = {n.name: s for n, s in asg.items()}
        self.apply_assignment(table, num_stage)
        return table

    def apply_assignment(self, table: Dict[str, int], num_stage: int) -> None:
        self.assignment = {n: table[n.name] for n in self.gm.graph.nodes}
        self.plan = build_stage_plan(self.gm, self.assignment, num_stage)
        self.metadata_range = [(s, f"submod_{s}") for s in range(num_stage)]
        self.special_nodes = self.cross_reference_analyze()

    def cross_reference_analyze(self) -> Dict[str, Tuple[int, int]]:
        """``{value: (producer stage, last consumer stage)}`` for every value that leaves its stage."""
        out: Dict[str, Tuple[int, int]] = {}
        by_name = {n.name: n for n in self.gm.graph.nodes}
        for b, names in enumerate(self.plan.cross):
            for name in names:
                src = self.assignment[by_name[name]]
                last = max(self.assignment[u] for u in by_name[name].users)
                out[name] = (src, last)
        return out

    # ---- per-stage module -------------------------------------------------------
    def setup_submod(self, stage: int) -> fx.GraphModule:
        self.stage = stage
        self.submod = extract_stage(self.gm, self.assignment, self.plan, stage)
        return self.submod

    def clean_module_memory(self) -> None:
        """Drop the whole-model graph; parameters of other stages lose their last reference here."""
        self.gm = None
        self.assignment = {}
        self.module = None

    def print_graph(self, rank: int = 0) -> None:
        if self.gm is not None:
            print(self.gm.graph)
