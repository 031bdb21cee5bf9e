"""Shape-aware torch.fx tracer for unmodified HuggingFace / nn.Module models.

The reference captures HF models with ``transformers.utils.fx.HFTracer``
(opt_prime/opt_prime/IR.py:1394-1440), which no longer exists in current
``transformers`` releases.  This tracer has no such dependency: every proxy
carries a *meta value* (a tensor on the ``meta`` device, or a plain Python
object) computed by running the recorded op on its arguments' meta values.
The graph stays symbolic in batch and sequence length (``x.shape``,
``x.size(1)``, ``x.device`` are nodes), while Python control flow that needs a
concrete answer (``if q.shape[2] > 1``, ``len(t)``, tuple unpacking,
``range(n)``) is resolved from the meta value, i.e. specialised to the example
inputs exactly where the model's own code branches on them.

Result: a module-level graph (``call_module`` for every leaf ``torch.nn``
module, ``call_function``/``call_method`` for the glue in between), which is the
form the partitioners, the tensor-parallel planner and the kernel rewrite pass
operate on.
"""
from __future__ import annotations

import builtins
import contextlib
import inspect
import math
import operator
import sys
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.fx as fx
import torch.nn as nn
from torch.fx.proxy import Attribute, Proxy

__all__ = ["MetaTracer", "trace_model", "TraceResult", "MODEL_TYPE_HF", "MODEL_TYPE_SYMBOLIC", "MODEL_TYPE_VIT"]

# Model-type tags select the name of the first placeholder, as in the
# reference (opt_prime/opt_prime/opti_pri.py:475, schedule.py:155-161).
MODEL_TYPE_HF = 50
MODEL_TYPE_SYMBOLIC = 51
MODEL_TYPE_VIT = 52

_UNKNOWN = object()

# Non-``torch.nn`` classes kept as single ``call_module`` nodes: they own
# buffers/parameters that are awkward as free ``get_attr`` nodes, and they are
# the units the kernel rewrite pass swaps for fused sm_100a implementations.
# "SparseMoeBlock": expert routing is data-dependent control flow (index lists per expert); the block is kept as one
# module call, which is also the unit the hierarchical partitioner groups by.
_DEFAULT_LEAF_SUFFIXES = ("RotaryEmbedding", "RMSNorm", "Conv1D", "SparseMoeBlock")
_SHAPE_PRESERVING_SUFFIXES = ("SparseMoeBlock",)

# Tensor factories do not dispatch through ``__torch_function__`` when only a
# size/device argument is a Proxy, so they are wrapped while tracing.
_FACTORY_NAMES = (
    "arange", "zeros", "ones", "full", "empty", "tensor", "eye", "linspace",
    "randn", "rand", "randint", "finfo", "iinfo",
)

# Mask builders of ``transformers`` are replaced while tracing (their vmap-based code cannot be traced).  With an
# attention implementation that derives causality itself (sdpa, flash) they return ``None`` and the causal structure
# is carried by ``is_causal`` of the attention op (the reference's export path does the same, IR.py:1582-1613).  The
# ``eager`` implementation has no other source of causality than the mask, so there the causal builders return a
# traceable additive mask ``[1, 1, q, q]`` built from ``arange`` comparisons on the embeddings' sequence length.
_MASK_BUILDERS = (
    "create_causal_mask", "create_sliding_window_causal_mask", "create_chunked_causal_mask",
    "create_bidirectional_mask", "create_masks_for_generate",
)
_CAUSAL_BUILDERS = ("create_causal_mask", "create_sliding_window_causal_mask", "create_chunked_causal_mask")


def _eager_causal_mask_builder(name: str):
    def build(*args, **kwargs):
        config = kwargs.get("config", args[0] if args else None)
        embeds = kwargs.get("inputs_embeds", kwargs.get("input_embeds"))
        if embeds is None:
            embeds = next((a for a in args[1:] if isinstance(a, (Proxy, torch.Tensor))), None)
        if embeds is None:
            return None
        q = embeds.shape[1]
        idx = torch.arange(q, device=embeds.device)
        keep = idx.unsqueeze(1) >= idx.unsqueeze(0)
        window = getattr(config, "sliding_window", None) if name == "create_sliding_window_causal_mask" else None
        if window:
            keep = keep & ((idx.unsqueeze(1) - idx.unsqueeze(0)) < window)
        mask = torch.zeros((q, q), dtype=embeds.dtype, device=embeds.device).masked_fill(~keep, torch.finfo(embeds.dtype).min)
        return mask.unsqueeze(0).unsqueeze(0)
    return build


def _has_proxy(obj: Any) -> bool:
    found = False

    def visit(a):
        nonlocal found
        if isinstance(a, Proxy):
            found = True
        return a

    fx.node.map_aggregate(obj, visit) if not isinstance(obj, Proxy) else visit(obj)
    return found


def _to_meta(v: Any) -> Any:
    if isinstance(v, torch.Tensor):
        return v if v.device.type == "meta" else v.detach().to("meta")
    if isinstance(v, (tuple, list)):
        out = [_to_meta(x) for x in v]
        if isinstance(v, torch.Size):
            return v
        try:
            return type(v)(out)
        except TypeError:
            return type(v)(*out)  # namedtuple
    if isinstance(v, dict):
        return {k: _to_meta(x) for k, x in v.items()}
    return v


class MetaProxy(Proxy):
    """Proxy whose node carries ``meta['val']``; concretises on Python demand."""

    def _val(self, what: str):
        v = self.node.meta.get("val", _UNKNOWN)
        if v is _UNKNOWN:
            raise fx.proxy.TraceError(
                f"{what} of '{self.node.name}' is needed while tracing but its value "
                f"could not be inferred from the example inputs")
        return v

    def __getattr__(self, k):
        if k.startswith("__") and k.endswith("__"):
            raise AttributeError(k)
        if k == "ndim":
            # the rank of a tensor is static: hand out the concrete value (``x.ndim == 3``).  ``dtype`` stays symbolic:
            # a model is traced in fp32 and may run in bf16, so no dtype of the trace may be baked into the graph
            # (``torch.finfo(x.dtype)`` is traced as a node, see the finfo / iinfo wrappers)
            v = self.node.meta.get("val", _UNKNOWN)
            if isinstance(v, torch.Tensor):
                return v.ndim
        return MetaAttribute(self, k)

    def __len__(self):
        return len(self._val("len()"))

    def __index__(self):
        return operator.index(self._val("an index"))

    def __int__(self):
        return int(self._val("int()"))

    def __float__(self):
        return float(self._val("float()"))

    def __contains__(self, item):
        return item in self._val("membership")

    def __hash__(self):
        return id(self)

    @property
    def __class__(self):  # keep isinstance(x, torch.Tensor) False, default Proxy behaviour
        return type(self)


class MetaAttribute(MetaProxy):
    """Lazy ``getattr`` node, mirroring ``torch.fx.proxy.Attribute``."""

    def __init__(self, root: Proxy, attr: str):
        self.root = root
        self.attr = attr
        self.tracer = root.tracer
        self._node: Optional[fx.Node] = None

    @property
    def node(self):
        if self._node is None:
            self._node = self.tracer.create_proxy("call_function", builtins.getattr, (self.root, self.attr), {}).node
        return self._node

    def __call__(self, *args, **kwargs):
        return self.tracer.create_proxy("call_method", self.attr, (self.root,) + args, kwargs)


class TraceResult:
    """Bundle returned by :func:`trace_model`."""

    def __init__(self, gm: fx.GraphModule, input_names: List[str], model_type: int):
        self.gm = gm
        self.input_names = input_names
        self.model_type = model_type


class MetaTracer(fx.Tracer):
    def __init__(self, leaf_classes: Sequence[str] = (), leaf_predicate: Optional[Callable[[nn.Module, str], bool]] = None,
                 autowrap_functions: Tuple[Callable, ...] = ()):
        super().__init__(autowrap_modules=(math,), autowrap_functions=autowrap_functions)
        self.leaf_classes = set(leaf_classes)
        self.leaf_predicate = leaf_predicate
        self._strip_prefix = ""
        self._meta_enabled = True
        self._in_meta_eval = 0
        self.proxy_buffer_attributes = True

    # ---- leaf policy -------------------------------------------------
    def is_leaf_module(self, m: nn.Module, qualname: str) -> bool:
        if type(m).__name__ in self.leaf_classes:
            return True
        if self.leaf_predicate is not None and self.leaf_predicate(m, qualname):
            return True
        if isinstance(m, (nn.Sequential, nn.ModuleList, nn.ModuleDict)):
            return False
        if type(m).__name__.endswith(_DEFAULT_LEAF_SUFFIXES):
            return True
        return m.__module__.startswith("torch.nn") or m.__module__.startswith("torch.ao.nn")

    def path_of_module(self, mod: nn.Module) -> str:
        p = super().path_of_module(mod)
        if self._strip_prefix and p.startswith(self._strip_prefix):
            p = p[len(self._strip_prefix):]
        return p

    # ---- proxies with meta values -------------------------------------
    def proxy(self, node: fx.Node) -> Proxy:
        return MetaProxy(node, self)

    def create_proxy(self, kind, target, args, kwargs, name=None, type_expr=None, proxy_factory_fn=None):
        if kind == "get_attr" and self._strip_prefix and isinstance(target, str) and target.startswith(self._strip_prefix):
            target = target[len(self._strip_prefix):]
        p = super().create_proxy(kind, target, args, kwargs, name, type_expr, proxy_factory_fn)
        if self._meta_enabled and kind != "placeholder":
            try:
                p.node.meta["val"] = self._infer_meta(kind, target, args, kwargs)
            except Exception as e:  # value unknown; only fatal if Python later demands it
                p.node.meta["val_error"] = repr(e)
        return p

    def _meta_of(self, a):
        def conv(x):
            if isinstance(x, Proxy):
                v = x.node.meta.get("val", _UNKNOWN)
                if v is _UNKNOWN:
                    raise RuntimeError(f"no meta value for {x.node.name}")
                return v
            return x
        if isinstance(a, Proxy):
            return conv(a)
        return fx.node.map_aggregate(a, conv)

    def _infer_meta(self, kind, target, args, kwargs):
        margs = self._meta_of(tuple(args))
        mkwargs = self._meta_of(dict(kwargs))
        self._in_meta_eval += 1
        try:
            return self._infer_meta_inner(kind, target, margs, mkwargs)
        finally:
            self._in_meta_eval -= 1

    def _infer_meta_inner(self, kind, target, margs, mkwargs):
        with torch.no_grad():
            if kind == "call_function":
                if target in _FACTORY_ORIGINALS.values() and getattr(target, "__name__", "") not in ("finfo", "iinfo"):
                    mkwargs = dict(mkwargs)
                    mkwargs["device"] = "meta"
                out = target(*margs, **mkwargs)
            elif kind == "call_method":
                self_obj, rest = margs[0], margs[1:]
                if target == "to" or target in ("cuda", "cpu"):
                    # device moves keep the value on meta
                    if target != "to":
                        return self_obj
                    rest = tuple("meta" if isinstance(r, (torch.device, str)) and not isinstance(r, torch.dtype) else r for r in rest)
                    if "device" in mkwargs:
                        mkwargs = dict(mkwargs, device="meta")
                out = getattr(self_obj, target)(*rest, **mkwargs)
            elif kind == "call_module":
                mod = self.root.get_submodule(self._strip_prefix + target if self._strip_prefix else target)
                state = {n: _to_meta(p) for n, p in list(mod.named_parameters()) + list(mod.named_buffers())}
                was_training = mod.training
                try:
                    out = torch.func.functional_call(mod, state, margs, mkwargs)
                except Exception:
                    # data-dependent routing cannot run on meta tensors; such blocks map the residual stream to a
                    # tensor of the same shape and dtype
                    first = next((a for a in margs if isinstance(a, torch.Tensor)), None)
                    if first is None or not type(mod).__name__.endswith(_SHAPE_PRESERVING_SUFFIXES):
                        raise
                    out = torch.empty_like(first)
                finally:
                    mod.train(was_training)
            elif kind == "get_attr":
                obj = self.root
                for part in (self._strip_prefix + target).split("."):
                    obj = getattr(obj, part)
                out = obj
            else:
                return _UNKNOWN
        return _to_meta(out)

    # ---- Python protocol hooks ------------------------------------------
    def to_bool(self, obj: Proxy) -> bool:
        v = obj.node.meta.get("val", _UNKNOWN)
        if v is _UNKNOWN:
            return super().to_bool(obj)
        if isinstance(v, torch.Tensor):
            raise fx.proxy.TraceError(f"data-dependent control flow on tensor '{obj.node.name}' cannot be traced")
        return bool(v)

    def iter(self, obj: Proxy):
        v = obj.node.meta.get("val", _UNKNOWN)
        if v is _UNKNOWN:
            return super().iter(obj)
        n = v.shape[0] if isinstance(v, torch.Tensor) else len(v)
        return iter([obj[i] for i in range(n)])

    def keys(self, obj: Proxy):
        v = obj.node.meta.get("val", _UNKNOWN)
        if isinstance(v, dict):
            return v.keys()
        return super().keys(obj)

    def call_module(self, m, forward, args, kwargs):
        if self._in_meta_eval:  # nested module calls of a meta evaluation are not recorded
            return forward(*args, **kwargs)
        return super().call_module(m, forward, args, kwargs)

    def getattr(self, attr, attr_val, parameter_proxy_cache):
        if self._in_meta_eval:
            return attr_val
        return super().getattr(attr, attr_val, parameter_proxy_cache)


_FACTORY_ORIGINALS: Dict[str, Callable] = {n: getattr(torch, n) for n in _FACTORY_NAMES if hasattr(torch, n)}


def _make_factory_wrapper(tracer: MetaTracer, orig: Callable):
    def wrapper(*args, **kwargs):
        if _has_proxy(args) or _has_proxy(kwargs):
            return tracer.create_proxy("call_function", orig, args, kwargs)
        return orig(*args, **kwargs)
    wrapper.__name__ = getattr(orig, "__name__", "factory")
    wrapper.__wrapped_factory__ = orig
    return wrapper


@contextlib.contextmanager
def _patched(tracer: MetaTracer, model: nn.Module, extra_patches: Dict[Tuple[Any, str], Any]):
    saved: List[Tuple[Any, str, Any]] = []

    def patch(obj, name, new):
        saved.append((obj, name, getattr(obj, name)))
        setattr(obj, name, new)

    try:
        for n, orig in _FACTORY_ORIGINALS.items():
            patch(torch, n, _make_factory_wrapper(tracer, orig))
        seen = set()
        for sub in model.modules():
            modname = type(sub).__module__
            if modname in seen or modname.startswith("torch."):
                continue
            seen.add(modname)
            pymod = sys.modules.get(modname)
            if pymod is None:
                continue
            eager = getattr(getattr(model, "config", None), "_attn_implementation", None) == "eager"
            for fn in _MASK_BUILDERS:
                if hasattr(pymod, fn):
                    patch(pymod, fn, _eager_causal_mask_builder(fn) if eager and fn in _CAUSAL_BUILDERS else (lambda *a, **k: None))
        for (obj, name), new in extra_patches.items():
            patch(obj, name, new)
        yield
    finally:
        for obj, name, old in reversed(saved):
            setattr(obj, name, old)


def _infer_model_type(model: nn.Module) -> int:
    cls = type(model)
    if cls.__module__.startswith("transformers."):
        if "vit" in cls.__name__.lower() or "pixel_values" in inspect.signature(model.forward).parameters and \
                "input_ids" not in inspect.signature(model.forward).parameters:
            return MODEL_TYPE_VIT
        return MODEL_TYPE_HF
    return MODEL_TYPE_SYMBOLIC


def _default_example(model: nn.Module, name: str, batch: int, seq: int):
    cfg = getattr(model, "config", None)
    if name in ("input_ids", "decoder_input_ids", "labels", "token_type_ids"):
        return torch.zeros(batch, seq, dtype=torch.long, device="meta")
    if name == "position_ids":
        return torch.zeros(batch, seq, dtype=torch.long, device="meta")
    if name == "attention_mask":
        return torch.ones(batch, seq, dtype=torch.long, device="meta")
    if name == "pixel_values":
        c = getattr(cfg, "num_channels", 3)
        s = getattr(cfg, "image_size", 224)
        return torch.zeros(batch, c, s, s, device="meta")
    if name == "input_features":
        return torch.zeros(batch, getattr(cfg, "num_mel_bins", 80), 2 * getattr(cfg, "max_source_positions", 1500), device="meta")
    raise ValueError(f"no default example for input '{name}'; pass example_inputs")


def trace_model(model: nn.Module, input_names: Optional[Sequence[str]] = None,
                example_inputs: Optional[Dict[str, torch.Tensor]] = None,
                leaf_classes: Sequence[str] = (), leaf_predicate=None,
                const_kwargs: Optional[Dict[str, Any]] = None,
                example_batch: int = 2, example_seq: int = 8,
                extra_patches: Optional[Dict[Tuple[Any, str], Any]] = None) -> TraceResult:
    """Trace ``model`` into a module-level ``GraphModule``.

    ``input_names`` are the forward arguments that become placeholders (default:
    ``input_ids`` for HF text models, ``pixel_values`` for vision models, the
    positional parameters for plain modules); every other argument keeps its
    default value, except that HF models get ``use_cache=False`` and
    ``return_dict=True`` (reference: IR.py:1502-1507).
    """
    model_type = _infer_model_type(model)
    sig = inspect.signature(model.forward)
    params = sig.parameters
    if input_names is None:
        if model_type == MODEL_TYPE_HF:
            if "input_ids" in params:
                input_names = ["input_ids"]
            elif "input_features" in params:
                input_names = ["input_features", "decoder_input_ids"]
            else:
                input_names = [next(iter(params))]
        elif model_type == MODEL_TYPE_VIT:
            input_names = ["pixel_values"]
        else:
            input_names = [n for n, p in params.items()
                           if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD) and p.default is p.empty]
    input_names = list(input_names)
    ckw = dict(const_kwargs or {})
    if model_type in (MODEL_TYPE_HF, MODEL_TYPE_VIT):
        has_var_kw = any(p.kind == p.VAR_KEYWORD for p in params.values())
        if "use_cache" in params:
            ckw.setdefault("use_cache", False)
        if "return_dict" in params or has_var_kw:
            ckw.setdefault("return_dict", True)

    examples = dict(example_inputs or {})
    symbolic_only = False
    for n in input_names:
        if n not in examples:
            if model_type == MODEL_TYPE_SYMBOLIC:
                # plain modules without examples: classic symbolic trace (no shape-dependent control flow allowed)
                symbolic_only = True
                break
            examples[n] = _default_example(model, n, example_batch, example_seq)
    examples = {k: _to_meta(v) for k, v in examples.items()}

    # Wrapper root with an explicit signature so that placeholders are exactly
    # ``input_names`` (fx cannot bind **kwargs of HF forwards).
    class _Root(nn.Module):
        def __init__(self, inner, ckw):
            super().__init__()
            self._m = inner
            self._ckw = ckw

    positional = model_type == MODEL_TYPE_SYMBOLIC
    call = ", ".join(input_names) if positional else ", ".join(f"{n}={n}" for n in input_names)
    src = f"def forward(self, {', '.join(input_names)}):\n    return self._m({call}, **self._ckw)\n"
    ns: Dict[str, Any] = {}
    exec(src, ns)  # noqa: S102 - generated from identifier names only
    for n in input_names:
        if not n.isidentifier():
            raise ValueError(f"bad input name {n!r}")
    _Root.forward = ns["forward"]
    root = _Root(model, ckw)

    tracer = MetaTracer(leaf_classes=leaf_classes, leaf_predicate=leaf_predicate)
    tracer._strip_prefix = "_m."
    tracer._meta_enabled = not symbolic_only

    # placeholders get their meta value from the examples
    orig_create_proxy = tracer.create_proxy

    def create_proxy(kind, target, args, kwargs, name=None, type_expr=None, proxy_factory_fn=None):
        p = orig_create_proxy(kind, target, args, kwargs, name, type_expr, proxy_factory_fn)
        if kind == "placeholder" and target in examples:
            p.node.meta["val"] = examples[target]
        return p

    tracer.create_proxy = create_proxy  # type: ignore[assignment]

    with _patched(tracer, model, extra_patches or {}):
        graph = tracer.trace(root)

    # Drop meta tensors that are not serialisable-cheap? They are tiny; keep
    # shapes/dtypes only to make the graph picklable across ranks.
    for node in graph.nodes:
        v = node.meta.pop("val", _UNKNOWN)
        if isinstance(v, torch.Tensor):
            node.meta["tensor_meta"] = (tuple(v.shape), v.dtype)
        node.meta.pop("val_error", None)
    gm = fx.GraphModule(model, graph, class_name=type(model).__name__)
    gm.graph.eliminate_dead_code()
    gm.recompile()
    return TraceResult(gm, input_names, model_type)
