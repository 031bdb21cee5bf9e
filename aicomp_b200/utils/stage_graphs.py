"""CUDA-graph capture of one pipeline stage's forward and backward, replayed per micro-batch.

A training step of a pipeline stage issues the same thousand-odd kernels for every micro-batch; launched from Python
they cost as much host time as they take on the device.  :class:`GraphedStage` captures the stage's forward (with the
loss on the last stage) and its backward into two CUDA graphs and replays them through an ``autograd.Function``, so
that a micro-batch costs two graph launches plus the copies into and out of the static buffers.

It differs from ``torch.cuda.make_graphed_callables`` where a pipeline needs it to:

* every slot (one per micro-batch that can be in flight) captures into a memory pool of its own.  Graphs that share a
  pool may re-use one another's transient blocks and must replay in capture order; a 1F1B schedule interleaves the
  slots (F0 F1 B0 F2 B1 ...), so a shared pool would let slot 0's forward overwrite what slot 1 saved for backward;
* warm-up and capture run on ONE side stream, so gradient-accumulator nodes created during warm-up belong to the
  capturing stream and the autograd engine has no second stream to order against (with two streams it records an
  event on the uncaptured one and the capture fails with ``cudaErrorStreamCaptureIsolation``);
* gradients handed back to autograd are copies of the static buffers: the pipeline sends input gradients
  asynchronously to the previous stage, and autograd may keep a parameter gradient as ``.grad``; the next replay of
  the slot must overwrite neither.

Parameters that accumulate into ``main_grad`` inside their own backward kernels return no gradient to autograd; any
other parameter's gradient comes back through the replay function and is accumulated into ``.grad`` by autograd as in
eager mode.  (The reference has no CUDA-graph path; it launches every kernel from Python each micro-batch,
opt_prime/opt_prime/schedule.py:250-340.)
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch

__all__ = ["GraphedStage", "capture_stage_slots"]


class _Replay(torch.autograd.Function):
    @staticmethod
    def forward(ctx, slot: "GraphedStage", n_args: int, *flat):
        for static, given in zip(slot.static_inputs, flat[:n_args]):
            if static.data_ptr() != given.data_ptr():
                static.copy_(given)
        slot.fwd_graph.replay()
        ctx.slot = slot
        ctx.n_args = n_args
        outs = tuple(o.detach() for o in slot.static_outputs)
        ctx.mark_non_differentiable(*(o for o, s in zip(outs, slot.static_outputs) if not s.requires_grad))
        return outs

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, *grads):
        slot: GraphedStage = ctx.slot
        for static, given in zip(slot.static_grad_outputs, grads):
            if static is None:
                continue
            if given is None:
                static.zero_()
            elif static.data_ptr() != given.data_ptr():
                static.copy_(given)
        slot.bwd_graph.replay()
        out: List[Optional[torch.Tensor]] = []
        it = iter(slot.static_grad_inputs)
        for i, t in enumerate(slot.diff_mask):
            if not t:
                out.append(None)
                continue
            g = next(it)
            if g is None:
                out.append(None)
            else:
                # always a copy: activation gradients leave through an asynchronous send while the slot replays again,
                # and autograd may adopt a parameter gradient as ``.grad`` itself, which the next replay would overwrite
                out.append(g.clone())
        return (None, None, *out)


class GraphedStage:
    """One captured instance ("slot") of ``fn(*args) -> tensor | tuple of tensors``.

    ``params`` are the parameters ``fn`` reads; they are passed to the replay function so that autograd sees the
    output depend on them.  ``__call__`` takes the same positional tensors as ``fn``.
    """

    def __init__(self, fn: Callable, sample_args: Sequence[torch.Tensor], params: Sequence[torch.nn.Parameter],
                 stream: torch.cuda.Stream, warmup: int = 2):
        self.params = [p for p in params if p.requires_grad]
        self.static_inputs = list(sample_args)
        self.n_args = len(self.static_inputs)
        surface = self.static_inputs + self.params
        self.diff_mask = [bool(t.requires_grad) for t in surface]
        diff = [t for t in surface if t.requires_grad]
        self.fwd_graph = torch.cuda.CUDAGraph()
        self.bwd_graph = torch.cuda.CUDAGraph()
        pool = torch.cuda.graph_pool_handle()

        def as_tuple(res) -> Tuple[torch.Tensor, ...]:
            return tuple(res) if isinstance(res, (tuple, list)) else (res,)

        torch.cuda.synchronize()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                outs = as_tuple(fn(*self.static_inputs))
                live = [o for o in outs if o.requires_grad]
                grads = torch.autograd.grad(live, diff, [torch.ones_like(o) for o in live], allow_unused=True)
                del outs, live, grads
        torch.cuda.synchronize()
        with torch.cuda.graph(self.fwd_graph, pool=pool, stream=stream, capture_error_mode="thread_local"):
            outs = as_tuple(fn(*self.static_inputs))
        self.static_outputs = outs
        self.static_grad_outputs = [torch.zeros_like(o) if o.requires_grad else None for o in outs]
        live = [o for o in outs if o.requires_grad]
        with torch.cuda.graph(self.bwd_graph, pool=pool, stream=stream, capture_error_mode="thread_local"):
            grads = torch.autograd.grad(live, diff, [g for g in self.static_grad_outputs if g is not None], allow_unused=True)
        self.static_grad_inputs = list(grads)
        self.single = len(outs) == 1

    def __call__(self, *args):
        outs = _Replay.apply(self, self.n_args, *args, *self.params)
        return outs[0] if self.single else outs


def capture_stage_slots(fn: Callable, make_sample: Callable[[], Sequence[torch.Tensor]],
                        params: Sequence[torch.nn.Parameter], n_slots: int) -> List[GraphedStage]:
    """``n_slots`` independent captures of ``fn`` (one per micro-batch in flight), all on one capture stream."""
    stream = torch.cuda.Stream()
    return [GraphedStage(fn, make_sample(), params, stream) for _ in range(n_slots)]
