"""Micro-batch pipeline schedules (GPipe and non-interleaved 1F1B).

Semantics follow the reference schedulers (opt_prime/opt_prime/schedule.py:
``ScheduleGPipe.run`` :965-1016, ``Schedule1F1B.run`` :1028-1125): the batch is
padded to a multiple of ``num_mb`` and chunked, every stage runs its module per
micro-batch with detached, grad-enabled boundary inputs, the last stage computes
the loss per micro-batch (mean over that micro-batch's tokens, not divided by
``num_mb``), data-parallel gradient reduction happens once after the last
micro-batch's backward, and stage-granular activation recomputation is optional.

What differs is the transport: receives for the next micro-batch are posted
before the current one computes and sends never block the compute stream, so
stage-to-stage copies over NVLink overlap the math (the reference's sends and
receives are blocking and serialised with compute).  A stage also returns
gradients for *every* differentiable tensor it received, not only the first.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn.functional as F

from ..utils.log import get_logger
from ..utils import nvtx

log = get_logger(__name__)

__all__ = ["Schedule", "ScheduleGPipe", "Schedule1F1B", "SCHEDULES"]


def _is_diff(t: Any) -> bool:
    return isinstance(t, torch.Tensor) and t.is_floating_point() and t.requires_grad


class Schedule:
    """Shared machinery; subclasses order the forward/backward micro-steps."""

    def __init__(self, engine):
        self.e = engine
        self.plan = engine.plan
        self.stage = engine.tpl.stage
        self.P = engine.tpl.pp_size
        self.M = engine.num_mb
        self.first = engine.tpl.is_first_stage()
        self.last = engine.tpl.is_last_stage()
        # per micro-batch state
        self.env: List[Dict[str, Any]] = []
        self.outs: List[Any] = []
        self.losses: List[Optional[torch.Tensor]] = []

    # ------------------------------------------------------------------ inputs
    def split_inputs(self, data, labels):
        M = self.M
        chunks: List[Dict[str, Any]] = [dict() for _ in range(M)]
        if self.first:
            if data is None:
                raise ValueError("the first pipeline stage needs the input batch")
            named = data if isinstance(data, dict) else {self.plan.input_names[0]: data}
            for k, v in named.items():
                if isinstance(v, torch.Tensor):
                    v = self.e._to_device(v)
                    if self.e.use_padding and v.shape[0] % M:
                        pad = M - v.shape[0] % M
                        v = torch.cat([v, v[-1:].expand(pad, *v.shape[1:])], 0)
                    parts = torch.chunk(v, M, 0)
                    if len(parts) != M:
                        raise ValueError(f"batch of {v.shape[0]} cannot be split into {M} micro-batches")
                    for i in range(M):
                        chunks[i][k] = parts[i]
                else:
                    for i in range(M):
                        chunks[i][k] = v
        label_chunks: List[Any] = [None] * M
        if self.last and labels is not None:
            if isinstance(labels, (list, tuple)) and len(labels) == M and isinstance(labels[0], torch.Tensor):
                label_chunks = [self.e._to_device(l) for l in labels]
            else:
                labels = self.e._to_device(labels)
                if self.e.use_padding and labels.shape[0] % M:
                    pad = M - labels.shape[0] % M
                    fill = torch.full((pad, *labels.shape[1:]), self.e.ignore_index, dtype=labels.dtype, device=labels.device)
                    labels = torch.cat([labels, fill], 0)
                label_chunks = list(torch.chunk(labels, M, 0))
        return chunks, label_chunks

    # ------------------------------------------------------------------ one forward micro-step
    def forward_step(self, mb: int, inputs: Dict[str, Any], labels) -> None:
        e = self.e
        with nvtx.range(f"F s{self.stage} mb{mb}"):
            env: Dict[str, Any] = {}
            if self.first:
                env.update(inputs)
            else:
                recv = e.fwd_in.wait_recv()
                env.update(dict(zip(self.plan.recv_names(self.stage), recv)))
                if mb + 1 < self.M:
                    e.fwd_in.post_recv(first=False)
            args = [env[n] for n in self.plan.stage_inputs[self.stage]]
            loss = None
            graphed = e.graphed_stage(mb, args, labels) if e.training else None
            if graphed is not None:
                # forward (and, on the last stage, the loss) replayed from a captured CUDA graph: two launches instead
                # of the thousand-odd kernel launches Python would issue for this micro-batch
                model_out = None
                res = graphed(*args, labels) if self.last else graphed(*args)
                res = res if isinstance(res, tuple) else (res,)
                if self.last:
                    loss, outs = res[0], res[1:]
                else:
                    outs = res
            elif e.activation_ckpt and not self.last:
                with torch.no_grad():
                    model_out, outs = e.stage_module(*args)
                for t in outs:  # recomputed in backward; downstream must still return gradients for them
                    if isinstance(t, torch.Tensor) and t.is_floating_point():
                        t.requires_grad_(True)
            else:
                model_out, outs = e.stage_module(*args)
            env.update(dict(zip(self.plan.stage_outputs[self.stage], outs)))
            if not self.last:
                payload = [env[n] for n in self.plan.send_names(self.stage)]
                e.fwd_out.send(payload, first=(mb == 0))
            if self.last and graphed is None:
                if labels is not None:
                    loss = e.loss_fn(model_out, labels)
                if e.preserve_output:
                    e.outputs[mb] = _detach_tree(model_out)
            self.env[mb] = env
            self.outs[mb] = None if self.last else (args if e.activation_ckpt else outs)
            self.losses[mb] = loss

    # ------------------------------------------------------------------ one backward micro-step
    def backward_step(self, mb: int) -> None:
        e = self.e
        with nvtx.range(f"B s{self.stage} mb{mb}"):
            env = self.env[mb]
            send_names = self.plan.send_names(self.stage)
            recv_names = self.plan.recv_names(self.stage)
            roots: List[torch.Tensor] = []
            root_grads: List[Optional[torch.Tensor]] = []
            relayed: List = []
            if self.last:
                loss = self.losses[mb]
                if loss is None:
                    raise RuntimeError("backward without labels on the last stage")
                roots.append(loss)
                root_grads.append(None)
            else:
                grads = e.bwd_in.wait_recv()
                if mb + 1 < self.M:
                    e.bwd_in.post_recv(first=False)
                if e.activation_ckpt:  # recompute this stage's forward with autograd on
                    args = self.outs[mb]
                    _, outs = e.stage_module(*args)
                    env.update(dict(zip(self.plan.stage_outputs[self.stage], outs)))
                gi = 0
                produced = set(self.plan.stage_outputs[self.stage])
                for n in send_names:
                    t = env[n]
                    if not _is_diff(t):
                        continue
                    g = grads[gi]
                    gi += 1
                    if n in produced:
                        roots.append(t)
                        root_grads.append(g)
                    else:
                        relayed.append((t, g))
            if roots:
                is_final = mb == self.order_last_backward
                with e.dp_sync_context(is_final):
                    torch.autograd.backward(roots, root_grads)
            if self.last and e.cuda_graphs:
                # a replayed graph writes its loss into one static tensor per slot: keep this micro-batch's value
                self.losses[mb] = self.losses[mb].detach().clone()
            for t, g in relayed:
                t.grad = g if t.grad is None else t.grad + g
            if not self.first:
                back = []
                for n in recv_names:
                    t = env[n]
                    if _is_diff(t):
                        back.append(t.grad if t.grad is not None else torch.zeros_like(t))
                e.bwd_out.send(back, first=(self.bwd_sent == 0))
                self.bwd_sent += 1
            self.env[mb] = None
            self.outs[mb] = None

    # ------------------------------------------------------------------ driver
    def order(self) -> List[tuple]:
        raise NotImplementedError

    def in_flight(self) -> int:
        """Largest number of micro-batches whose forward has run and whose backward has not."""
        raise NotImplementedError

    def run(self, data, labels) -> None:
        e = self.e
        M = self.M
        self.env = [None] * M
        self.outs = [None] * M
        self.losses = [None] * M
        self.bwd_sent = 0
        e.outputs = [None] * M
        chunks, label_chunks = self.split_inputs(data, labels)
        import os as _os
        import time as _time
        prof = StepProfile(e.device) if _os.environ.get("AICOMP_PROFILE_SCHEDULE") == "1" else None
        t_run0 = _time.perf_counter()
        steps = self.order()
        self.order_last_backward = [mb for kind, mb in steps if kind == "B"][-1] if e.training else -1
        if not self.first:
            e.fwd_in.post_recv(first=True)
        posted_bwd = False
        for kind, mb in steps:
            tok = prof.begin() if prof else None
            if kind == "F":
                self.forward_step(mb, chunks[mb], label_chunks[mb])
            else:
                if not self.last and not posted_bwd:
                    e.bwd_in.post_recv(first=True)
                    posted_bwd = True
                self.backward_step(mb)
            if prof:
                prof.end(kind, tok)
        for ch in (e.fwd_out, e.bwd_out):
            if ch is not None:
                ch.flush()
        e.losses = self.losses
        if e.training:
            e.dp_finish()
        if prof:
            out = prof.summary()
            out["wall_ms"] = round(1e3 * (_time.perf_counter() - t_run0), 1)
            print(f"[schedule profile] rank {e.comm.rank} stage {self.stage}: {out}", flush=True)


def _detach_tree(x):
    if isinstance(x, torch.Tensor):
        return x.detach()
    if isinstance(x, dict):
        return {k: _detach_tree(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_detach_tree(v) for v in x)
    return x


class ScheduleGPipe(Schedule):
    """All forwards, then all backwards."""

    def in_flight(self) -> int:
        return self.M

    def order(self):
        steps = [("F", i) for i in range(self.M)]
        if self.e.training:
            steps += [("B", i) for i in range(self.M)]
        return steps


class Schedule1F1B(Schedule):
    """Warm-up of ``P-1-stage`` forwards, then one-forward-one-backward, then the remaining backwards."""

    def in_flight(self) -> int:
        return max(1, min(self.P - self.stage, self.M))

    def order(self):
        if not self.e.training:
            return [("F", i) for i in range(self.M)]
        warm = min(self.P - 1 - self.stage, self.M)
        steps = [("F", i) for i in range(warm)]
        f, b = warm, 0
        while f < self.M:
            steps.append(("F", f)); f += 1
            steps.append(("B", b)); b += 1
        while b < self.M:
            steps.append(("B", b)); b += 1
        return steps


SCHEDULES = {"gpipe": ScheduleGPipe, "1f1b": Schedule1F1B}


class StepProfile:
    """Optional per-step breakdown (``AICOMP_PROFILE_SCHEDULE=1``): device time inside forward / backward micro-steps
    (CUDA events), host time spent issuing them, and the step's wall time, printed per rank."""

    def __init__(self, device):
        self.cuda = device.type == "cuda"
        self.ev = []
        self.host = {"F": 0.0, "B": 0.0}

    def begin(self):
        import time
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
        else:
            e = None
        return e, time.perf_counter()

    def end(self, kind, tok):
        import time
        e0, t0 = tok
        self.host[kind] += time.perf_counter() - t0
        if self.cuda:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            self.ev.append((kind, e0, e1))

    def summary(self):
        dev = {"F": 0.0, "B": 0.0}
        if self.cuda:
            torch.cuda.synchronize()
            for k, a, b in self.ev:
                dev[k] += a.elapsed_time(b)
        return {"dev_F_ms": round(dev["F"], 1), "dev_B_ms": round(dev["B"], 1), "host_F_ms": round(1e3 * self.host["F"], 1),
                "host_B_ms": round(1e3 * self.host["B"], 1)}
