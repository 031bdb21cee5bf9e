"""Graph capture through ``torch.export`` (``dynamo_capture=True``), rebuilt as a module-level graph.

The reference's second capture path exports the model to ATen IR and regroups ATen nodes into module calls from
``nn_module_stack`` metadata, with a series of fix-ups for mismatching signatures
(opt_prime/opt_prime/IR.py:293-921, 1443-1744).  Here the regrouping is delegated to the exporter itself:

1. ``torch.export.export(strict=False)`` with dynamic batch / sequence dimensions, ``use_cache=False`` forced and the
   HF mask builders replaced by ``None`` (the causal structure lives in ``is_causal``);
2. ``torch.export.unflatten`` rebuilds the module hierarchy as nested graph modules;
3. that hierarchy is flattened again into ONE ``fx.Graph`` over the *original* model: containers are inlined; a leaf
   module (``torch.nn`` leaves, norm classes) whose exported call still binds to its original ``forward`` becomes a
   ``call_module`` node on the original module object, any other module is inlined as ATen ops (the reference
   "demotes" such modules the same way, IR.py:444-482); parameters used inline become ``get_attr`` nodes on the
   original model, and the ATen glue between modules is copied as is.

The result has the same form as :func:`aicomp_b200.graph.tracer.trace_model` produces, so the kernel rewrite pass,
the partitioners and the stage extraction apply unchanged.
"""
from __future__ import annotations

import inspect
import sys
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.fx as fx
import torch.nn as nn

from .tracer import (_CAUSAL_BUILDERS, _DEFAULT_LEAF_SUFFIXES, _MASK_BUILDERS, MODEL_TYPE_HF, MODEL_TYPE_SYMBOLIC, MODEL_TYPE_VIT,
                     TraceResult, _default_example, _eager_causal_mask_builder, _infer_model_type)

__all__ = ["export_to_module_graph"]


def _is_leaf(m: nn.Module, leaf_classes: Sequence[str]) -> bool:
    name = type(m).__name__
    if name in leaf_classes or name.endswith(_DEFAULT_LEAF_SUFFIXES):
        return True
    if isinstance(m, (nn.Sequential, nn.ModuleList, nn.ModuleDict)):
        return False
    return m.__module__.startswith("torch.nn")


def _leaf_paths(model: nn.Module, leaf_classes: Sequence[str]) -> List[str]:
    out: List[str] = []

    def walk(mod: nn.Module, prefix: str):
        for name, child in mod.named_children():
            path = f"{prefix}.{name}" if prefix else name
            if _is_leaf(child, leaf_classes):
                out.append(path)
            else:
                walk(child, path)
    walk(model, "")
    return out


class _Flattener:
    def __init__(self, model: nn.Module, unflat: nn.Module, leaves: Sequence[str]):
        self.model, self.unflat = model, unflat
        self.leaves = set(leaves)
        self.graph = fx.Graph()
        self.used_names: Dict[str, int] = {}

    def _name(self, base: str) -> str:
        base = base.replace(".", "_")
        n = self.used_names.get(base, 0)
        self.used_names[base] = n + 1
        return base if n == 0 else f"{base}_{n}"

    def inline(self, mod: nn.Module, prefix: str, args: tuple, kwargs: dict):
        g: fx.Graph = mod.graph
        env: Dict[fx.Node, Any] = {}
        placeholders = [n for n in g.nodes if n.op == "placeholder"]
        flat_args = list(args)
        for i, ph in enumerate(placeholders):
            if i < len(flat_args):
                env[ph] = flat_args[i]
            elif ph.target in kwargs:
                env[ph] = kwargs[ph.target]
            elif ph.name in kwargs:
                env[ph] = kwargs[ph.name]
            else:
                env[ph] = None
        result = None
        for node in g.nodes:
            if node.op == "placeholder":
                continue
            if node.op == "output":
                result = fx.node.map_arg(node.args[0], lambda n: env[n])
                continue
            a = fx.node.map_arg(node.args, lambda n: env[n])
            k = fx.node.map_arg(node.kwargs, lambda n: env[n])
            if node.op == "call_module":
                path = f"{prefix}.{node.target}" if prefix else str(node.target)
                child = mod.get_submodule(str(node.target))
                if path in self.leaves and self._single_output(child) and self._signature_ok(path, a, k):
                    new = self.graph.call_module(path, a, k)
                    new.name = self._name(path)
                    new.meta = dict(node.meta)
                    env[node] = new
                else:
                    env[node] = self.inline(child, path, a, k)
            elif node.op == "get_attr":
                path = f"{prefix}.{node.target}" if prefix else str(node.target)
                new = self.graph.get_attr(self._resolve_attr(path, mod, str(node.target)))
                new.meta = dict(node.meta)
                env[node] = new
            else:
                new = self.graph.create_node(node.op, node.target, a, k, name=self._name(node.name))
                new.meta = dict(node.meta)
                env[node] = new
        return result

    @staticmethod
    def _single_output(child: nn.Module) -> bool:
        """The exported sub-graph must return exactly one value, as the original module does; exported modules that also
        hand out intermediates (values the surrounding code re-uses) cannot be swapped for the original."""
        g = getattr(child, "graph", None)
        if g is None:
            return False
        out = next(n for n in g.nodes if n.op == "output").args[0]
        return isinstance(out, fx.Node)

    def _signature_ok(self, path: str, a: tuple, k: dict) -> bool:
        """The exporter passes a module only the tensors it really consumes (and sometimes symbolic sizes in front).
        The call is kept as a module call when it binds to the original ``forward`` with tensor arguments only and
        fills every required parameter; anything else is inlined as ATen ops."""
        try:
            fwd = self.model.get_submodule(path).forward
            bound = inspect.signature(fwd).bind(*a, **k)
        except (TypeError, AttributeError):
            return False
        for v in list(bound.args) + list(bound.kwargs.values()):
            if isinstance(v, fx.Node):
                val = v.meta.get("val")
                if val is not None and not isinstance(val, torch.Tensor):
                    return False  # a SymInt carrier, not a real argument of the module
        return True

    def _resolve_attr(self, path: str, owner: nn.Module, local: str) -> str:
        """Attribute path on the ORIGINAL model; constants that exist only in the exported program are copied over."""
        obj: Any = self.model
        try:
            for part in path.split("."):
                obj = getattr(obj, part)
            if isinstance(obj, torch.Tensor):
                return path
        except AttributeError:
            pass
        val = owner
        for part in local.split("."):
            val = getattr(val, part)
        name = "exported_const_" + path.replace(".", "_")
        if not hasattr(self.model, name):
            if isinstance(val, torch.Tensor):
                self.model.register_buffer(name, val.detach(), persistent=False)
            else:
                setattr(self.model, name, val)
        return name


def export_to_module_graph(model: nn.Module, input_names: Optional[Sequence[str]] = None,
                           example_inputs: Optional[Dict[str, torch.Tensor]] = None, leaf_classes: Sequence[str] = (),
                           example_batch: int = 2, example_seq: int = 16) -> TraceResult:
    model_type = _infer_model_type(model)
    params = inspect.signature(model.forward).parameters
    if input_names is None:
        if model_type == MODEL_TYPE_HF:
            input_names = ["input_ids"] if "input_ids" in params else [next(iter(params))]
        elif model_type == MODEL_TYPE_VIT:
            input_names = ["pixel_values"]
        else:
            input_names = [n for n, p in params.items() if p.default is p.empty and p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    input_names = list(input_names)
    examples = dict(example_inputs or {})
    device = next((p.device for p in model.parameters()), torch.device("cpu"))
    for n in input_names:
        if n not in examples:
            if model_type == MODEL_TYPE_SYMBOLIC:
                raise ValueError("example_inputs are required to export a plain nn.Module")
            ex = _default_example(model, n, max(example_batch, 2), example_seq)  # batch >= 2 avoids 0/1 specialisation
            examples[n] = torch.zeros(ex.shape, dtype=ex.dtype, device=device)
    kwargs: Dict[str, Any] = dict(examples)
    dyn: Dict[str, Any] = {}
    from torch.export import Dim
    batch = Dim("batch", min=1, max=256)
    max_pos = int(getattr(getattr(model, "config", None), "max_position_embeddings", 2048))
    seq = Dim("seq", min=2, max=max(3, max_pos - 1))
    for n, t in examples.items():
        if t.dim() >= 2 and t.dtype in (torch.int64, torch.int32) and model_type == MODEL_TYPE_HF:
            dyn[n] = {0: batch, 1: seq}
        elif t.dim() >= 1:
            dyn[n] = {0: batch}
        else:
            dyn[n] = None
    if model_type in (MODEL_TYPE_HF, MODEL_TYPE_VIT) and "use_cache" in params:
        kwargs["use_cache"] = False
        dyn["use_cache"] = None
    leaves = _leaf_paths(model, leaf_classes)
    saved = []
    try:
        seen = set()
        for sub in model.modules():
            pm = sys.modules.get(type(sub).__module__)
            if pm is None or pm.__name__ in seen or pm.__name__.startswith("torch."):
                continue
            seen.add(pm.__name__)
            eager = getattr(getattr(model, "config", None), "_attn_implementation", None) == "eager"
            for fn in _MASK_BUILDERS:
                if hasattr(pm, fn):
                    saved.append((pm, fn, getattr(pm, fn)))
                    # eager attention has no other source of causality than the mask: give it a traceable one
                    setattr(pm, fn, _eager_causal_mask_builder(fn) if eager and fn in _CAUSAL_BUILDERS else (lambda *a, **k: None))
        positional = model_type == MODEL_TYPE_SYMBOLIC
        ep = torch.export.export(model, tuple(examples[n] for n in input_names) if positional else (),
                                 {} if positional else kwargs,
                                 dynamic_shapes=(tuple(dyn[n] for n in input_names) if positional else dyn), strict=False)
    finally:
        for pm, fn, old in saved:
            setattr(pm, fn, old)
    unflat = torch.export.unflatten(ep)
    fl = _Flattener(model, unflat, leaves)
    root_placeholders = [n for n in unflat.graph.nodes if n.op == "placeholder"]
    args = []
    for ph in root_placeholders:
        if str(ph.target) in input_names:
            node = fl.graph.placeholder(str(ph.target))
            node.meta = dict(ph.meta)
            args.append(node)
        else:
            args.append(kwargs.get(str(ph.target)))  # constant keyword (e.g. use_cache=False)
    out = fl.inline(unflat, "", tuple(args), {})
    # HF models return a ModelOutput; the engine expects a dict with 'logits' (as the tracer produces)
    result = _restructure_output(out, model_type)
    fl.graph.output(result)
    for node in fl.graph.nodes:
        v = node.meta.pop("val", None)
        node.meta = {k: m for k, m in node.meta.items() if k in ("tensor_meta",)}
        if isinstance(v, torch.Tensor):
            try:
                node.meta["tensor_meta"] = (tuple(int(d) for d in v.shape), v.dtype)
            except Exception:
                pass
    gm = fx.GraphModule(model, fl.graph, class_name=type(model).__name__)
    gm.graph.eliminate_dead_code()
    gm.recompile()
    return TraceResult(gm, input_names, model_type)


def _restructure_output(flat_out, model_type: int) -> Any:
    """HF heads return a ``ModelOutput`` whose first exported leaf is the logits: hand the engine ``{'logits': ...}`` as
    the tracer does; plain modules return their tensor (or tuple) unchanged."""
    leaves = [v for v in (list(flat_out) if isinstance(flat_out, (tuple, list)) else [flat_out]) if v is not None]
    if model_type in (MODEL_TYPE_HF, MODEL_TYPE_VIT):
        return {"logits": leaves[0]}
    return leaves[0] if len(leaves) == 1 else tuple(leaves)
