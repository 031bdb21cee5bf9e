"""Stage extraction and cross-stage dataflow analysis.

Given a traced graph and a ``{node: stage}`` assignment this builds, for the
local stage only, a ``GraphModule`` that owns just the parameters it uses (the
other stages' weights are never materialised on this rank - the role of
``clean_module_memory`` in the reference, opt_prime/opt_prime/IR.py:2908-3013),
and the boundary tables the runtime needs:

``cross[b]``  ordered names of all values produced on a stage <= b (model
              inputs count as stage 0) and consumed on a stage > b.  Stage s
              receives ``cross[s-1]`` from s-1 and sends ``cross[s]`` to s+1;
              a value that skips stages is relayed hop by hop, like the
              reference's ``special_nodes`` (IR.py:2754-2828).

Module paths keep their dotted HF names inside the stage module, so a stage
``state_dict`` uses real parameter names; the reference's flattened
``moved_*`` names exist only at the checkpoint boundary.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

import torch
import torch.fx as fx
import torch.nn as nn

__all__ = ["StagePlan", "build_stage_plan", "extract_stage"]


@dataclass
class StagePlan:
    num_stage: int
    input_names: List[str]                         # model inputs (placeholders), in order
    cross: List[List[str]]                         # cross[b] for b in 0..num_stage-2
    stage_inputs: List[List[str]]                  # values each stage module takes (subset of env), in order
    stage_outputs: List[List[str]]                 # values each stage module returns besides the model output
    has_model_output: List[bool]                   # True for the stage that returns the model's output
    node_stage: Dict[str, int] = field(default_factory=dict)
    modules_per_stage: List[List[str]] = field(default_factory=list)

    def recv_names(self, stage: int) -> List[str]:
        return [] if stage == 0 else self.cross[stage - 1]

    def send_names(self, stage: int) -> List[str]:
        return [] if stage >= self.num_stage - 1 else self.cross[stage]


def build_stage_plan(gm: fx.GraphModule, assignment: Dict[fx.Node, int], num_stage: int) -> StagePlan:
    order = {n: i for i, n in enumerate(gm.graph.nodes)}
    input_names = [n.name for n in gm.graph.nodes if n.op == "placeholder"]
    last_use_stage: Dict[fx.Node, int] = {}
    for n in gm.graph.nodes:
        for a in n.all_input_nodes:
            last_use_stage[a] = max(last_use_stage.get(a, -1), assignment[n])
    cross: List[List[str]] = []
    for b in range(num_stage - 1):
        names = [n.name for n in gm.graph.nodes
                 if n.op != "output" and assignment[n] <= b and last_use_stage.get(n, -1) > b]
        cross.append(names)
    stage_inputs: List[List[str]] = []
    stage_outputs: List[List[str]] = []
    has_out: List[bool] = []
    mods: List[List[str]] = []
    for s in range(num_stage):
        mine = [n for n in gm.graph.nodes if assignment[n] == s and n.op not in ("placeholder", "output")]
        mine_set = set(mine)
        ins: List[fx.Node] = []
        for n in mine + [o for o in gm.graph.nodes if o.op == "output" and assignment[o] == s]:
            for a in n.all_input_nodes:
                if a not in mine_set and a not in ins:
                    ins.append(a)
        ins.sort(key=lambda a: order[a])
        stage_inputs.append([a.name for a in ins])
        outs = [n.name for n in mine if last_use_stage.get(n, -1) > s]
        stage_outputs.append(outs)
        has_out.append(any(o.op == "output" and assignment[o] == s for o in gm.graph.nodes))
        mods.append([str(n.target) for n in mine if n.op == "call_module"])
    return StagePlan(num_stage, input_names, cross, stage_inputs, stage_outputs, has_out,
                     {n.name: assignment[n] for n in gm.graph.nodes}, mods)


class _StageModule(fx.GraphModule):
    """GraphModule of one pipeline stage: ``forward(*stage_inputs) -> (model_output | None, stage_outputs...)``."""


def extract_stage(gm: fx.GraphModule, assignment: Dict[fx.Node, int], plan: StagePlan, stage: int) -> fx.GraphModule:
    """Copy the nodes of ``stage`` into a fresh graph; only the referenced submodules/attributes are kept."""
    g = fx.Graph()
    env: Dict[fx.Node, fx.Node] = {}
    by_name = {n.name: n for n in gm.graph.nodes}
    for name in plan.stage_inputs[stage]:
        src = by_name[name]
        ph = g.placeholder(name)
        ph.meta = dict(src.meta)
        env[src] = ph
    model_out = None
    for n in gm.graph.nodes:
        if n.op == "placeholder":
            continue
        if n.op == "output":
            if assignment[n] == stage:
                model_out = fx.node.map_arg(n.args[0], lambda a: env[a])
            continue
        if assignment[n] != stage:
            continue
        env[n] = g.node_copy(n, lambda a: env[a])
    outs = tuple(env[by_name[name]] for name in plan.stage_outputs[stage])
    g.output((model_out, outs))
    g.lint()
    sm = fx.GraphModule(gm, g, class_name=f"Stage{stage}")
    return sm
