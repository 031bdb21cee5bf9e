"""Fused AdamW over a flat parameter arena (bf16 weights, fp32 master weights and moments).

Layout for 180 GB HBM3e: all parameters of a pipeline stage live in ONE bf16
buffer; master weights, both moments and the fp32 main gradient are parallel
flat buffers (16 bytes of state + 2 bytes of weight per parameter).  Consequences:

* the optimizer step is a single kernel over the arena (``b200_adamw``), which also
  zeroes the gradient for the next step;
* weight-gradient GEMMs accumulate straight into the fp32 main gradient
  (``param.main_grad`` views), so micro-batch accumulation costs no extra pass
  and loses no precision;
* the data-parallel reducer works on contiguous slices of the gradient arena,
  with no flatten/unflatten copies;
* global-norm clipping is one reduction kernel plus a device scalar that the
  update kernel reads - no host synchronisation.

The reference leaves the optimizer to user code (``torch.optim.Adam`` on fp32
parameters, opt_prime/examples/pp_train_llama5.py:134); this class is a drop-in
``torch.optim.Optimizer`` for that role.  On CPU (or fp32 parameters) it
delegates to ``torch.optim.AdamW`` so the same script runs in tests.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from .. import ops

__all__ = ["FusedAdamW"]

_ALIGN = 128  # elements; keeps every parameter 256-byte aligned inside the arena (TMA needs 16)


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 grad_scale: float = 1.0, max_grad_norm: float = 0.0, norm_groups: Optional[Dict[str, Any]] = None):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.grad_scale = float(grad_scale)
        self.max_grad_norm = float(max_grad_norm)
        self.norm_groups = norm_groups or {}
        self._step = 0
        self._grad_is_zero = True
        all_params = [p for g in self.param_groups for p in g["params"]]
        self.fused = bool(all_params) and all(p.is_cuda and p.dtype == torch.bfloat16 for p in all_params)
        self._fallback: Optional[torch.optim.AdamW] = None
        if not self.fused:
            self._fallback = torch.optim.AdamW(self.param_groups, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
            return
        _lib.require()
        dev = all_params[0].device
        # TP-sharded parameters first, replicated ones after: the squared norm of each part reduces differently
        order: List[torch.nn.Parameter] = []
        self._group_ranges = []
        for g in self.param_groups:
            ps = sorted(g["params"], key=lambda p: 0 if getattr(p, "tp_sharded", False) else 1)
            start = sum(_pad(p.numel()) for p in order)
            order.extend(ps)
            self._group_ranges.append((start, sum(_pad(p.numel()) for p in order)))
        self._order = order
        total = sum(_pad(p.numel()) for p in order)
        self.p16 = torch.zeros(total, dtype=torch.bfloat16, device=dev)
        self.offsets: List[int] = []
        off = 0
        n_sharded = 0
        for p in order:
            n = p.numel()
            self.offsets.append(off)
            self.p16[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.p16[off:off + n].view(p.shape)
            off += _pad(n)
            if getattr(p, "tp_sharded", False) and len(self.param_groups) == 1:
                n_sharded = off
        self._sharded_end = n_sharded
        self.master = self.p16.float()
        self.m = torch.zeros(total, dtype=torch.float32, device=dev)
        self.v = torch.zeros(total, dtype=torch.float32, device=dev)
        self.grad = torch.zeros(total, dtype=torch.float32, device=dev)
        for p, o in zip(order, self.offsets):
            p.main_grad = self.grad[o:o + p.numel()].view(p.shape)
            p.grad_accumulated = False
        self._norm_sq = torch.zeros(2, dtype=torch.float32, device=dev)
        self.total = total
        # data-parallel sharding of the optimizer state (set by attach_to_reducer): this rank updates [lo, hi) only
        self.shard = (0, total)
        self._dp_group = None

    # ------------------------------------------------------------------ gradient plumbing
    def _fold_param_grads(self) -> None:
        """Gradients that autograd produced in ``.grad`` (ops without main-grad fusion) are added to the arena."""
        lib = _lib.require()
        for p, o in zip(self._order, self.offsets):
            g = p.grad
            if g is None:
                continue
            n = p.numel()
            dst = self.grad[o:o + n]
            if g.dtype == torch.bfloat16 and g.is_contiguous() and n % 4 == 0:
                _lib.check_rc(lib.b200_accum_bf16_f32(g.data_ptr(), dst.data_ptr(), n, _lib.stream_ptr()), "accum")
            else:
                dst.add_(g.reshape(-1).float())
            p.grad = None

    def attach_to_reducer(self, reducer, shard_state: bool = True) -> None:
        """Let a data-parallel ``GradReducer`` reduce the contiguous gradient arena in place.

        ``shard_state`` (default): the optimizer state is sharded over the data-parallel group.  The reducer then only
        reduce-scatters the gradient arena, every rank keeps master weights and moments for its own 1/dp slice, updates
        that slice, and the bf16 weights are all-gathered after the update.  Per step this moves 3/4 of the bytes of
        an all-reduce of the fp32 gradients and runs the update kernel over 1/dp of the parameters.
        """
        if not (self.fused and reducer is not None):
            return
        dp = reducer.dp_size
        shard = bool(shard_state) and dp > 1 and self._step == 0
        if shard and self.total % (8 * dp):   # equal 16-byte aligned slices for the all-gather of the weights
            self._repad(((self.total + 8 * dp - 1) // (8 * dp)) * 8 * dp)
        fused = getattr(reducer, "_fused", None)
        if fused is not None:  # move the gradient arena into peer-mapped memory (collective over the DP group)
            new = fused.alloc_arena(self.total)
            new.copy_(self.grad)
            self.grad = new
            for p, o in zip(self._order, self.offsets):
                p.main_grad = self.grad[o:o + p.numel()].view(p.shape)
        reducer.arena_grad = self.grad
        reducer.pre_reduce = self._fold_param_grads
        if shard:
            lo, hi = reducer.shard_bounds(self.total)
            self.shard = (lo, hi)
            self._dp_group = reducer.group
            self.master = self.p16[lo:hi].float()
            self.m = torch.zeros(hi - lo, dtype=torch.float32, device=self.p16.device)
            self.v = torch.zeros(hi - lo, dtype=torch.float32, device=self.p16.device)
            reducer.arena_mode = "reduce_scatter"

    def _repad(self, new_total: int) -> None:
        """Grow the flat buffers to ``new_total`` elements (tail padding), keeping every parameter where it is."""
        dev = self.p16.device
        p16 = torch.zeros(new_total, dtype=torch.bfloat16, device=dev)
        p16[:self.total].copy_(self.p16)
        self.p16 = p16
        grad = torch.zeros(new_total, dtype=torch.float32, device=dev)
        grad[:self.total].copy_(self.grad)
        self.grad = grad
        for p, o in zip(self._order, self.offsets):
            p.data = self.p16[o:o + p.numel()].view(p.shape)
            p.main_grad = self.grad[o:o + p.numel()].view(p.shape)
        self.master = self.p16.float()
        self.m = torch.zeros(new_total, dtype=torch.float32, device=dev)
        self.v = torch.zeros(new_total, dtype=torch.float32, device=dev)
        if self._group_ranges:
            lo, _ = self._group_ranges[-1]
            self._group_ranges[-1] = (lo, new_total)
        self.total = new_total
        self.shard = (0, new_total)

    def grad_norm(self) -> torch.Tensor:
        """Global L2 norm of the (unscaled) gradient; reduces over the ``tp`` / ``pp`` groups given in ``norm_groups``."""
        if not self.fused:
            ps = [p.grad.detach().float().pow(2).sum() for g in self.param_groups for p in g["params"] if p.grad is not None]
            return torch.stack(ps).sum().sqrt() if ps else torch.zeros(())
        self._fold_param_grads()
        return self._compute_norm_sq().sqrt()

    def _compute_norm_sq(self) -> torch.Tensor:
        lib = _lib.require()
        self._norm_sq.zero_()
        se = self._sharded_end
        lo, hi = self.shard   # with a sharded optimizer only this rank's slice holds reduced gradients
        a0, a1 = lo, min(hi, se)
        if a1 > a0:
            _lib.check_rc(lib.b200_sumsq(self.grad[a0:].data_ptr(), a1 - a0, self._norm_sq[0:1].data_ptr(), _lib.stream_ptr()), "sumsq")
        b0, b1 = max(lo, se), hi
        if b1 > b0:
            _lib.check_rc(lib.b200_sumsq(self.grad[b0:].data_ptr(), b1 - b0, self._norm_sq[1:2].data_ptr(), _lib.stream_ptr()), "sumsq")
        if self._dp_group is not None:
            dist.all_reduce(self._norm_sq, group=self._dp_group)
        tp, pp = self.norm_groups.get("tp"), self.norm_groups.get("pp")
        if tp is not None:
            dist.all_reduce(self._norm_sq[0:1], group=tp)
        total = self._norm_sq.sum(0, keepdim=True)
        if pp is not None:
            dist.all_reduce(total, group=pp)
        return total

    # ------------------------------------------------------------------ Optimizer API
    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        if not self.fused:
            self._fallback.step()
            return loss
        self._fold_param_grads()
        self._step += 1
        lib = _lib.require()
        norm_ptr = None
        if self.max_grad_norm > 0:
            self._norm_total = self._compute_norm_sq()  # kept alive until the update kernel has read it
            norm_ptr = self._norm_total.data_ptr()
        s_lo, s_hi = self.shard
        for g, (g_lo, g_hi) in zip(self.param_groups, self._group_ranges):
            lo, hi = max(g_lo, s_lo), min(g_hi, s_hi)
            if hi <= lo:
                continue
            b1, b2 = g["betas"]
            so = lo - s_lo   # master weights and moments exist for this rank's slice only
            rc = lib.b200_adamw(self.p16[lo:].data_ptr(), self.master[so:].data_ptr(), self.m[so:].data_ptr(), self.v[so:].data_ptr(),
                                self.grad[lo:].data_ptr(), None, norm_ptr, hi - lo, float(g["lr"]), float(b1), float(b2),
                                float(g["eps"]), float(g["weight_decay"]), self._step, self.grad_scale, self.max_grad_norm, 1,
                                _lib.stream_ptr())
            _lib.check_rc(rc, "adamw")
            ops._count()
        if self._dp_group is not None:
            # the update kernel cleared the gradient of this slice; the other slices hold this rank's unreduced values
            if s_lo > 0:
                self.grad[:s_lo].zero_()
            if s_hi < self.total:
                self.grad[s_hi:].zero_()
            dist.all_gather_into_tensor(self.p16, self.p16[s_lo:s_hi], group=self._dp_group)
        self._grad_is_zero = True
        for p in self._order:
            p.grad_accumulated = False
        return loss

    def zero_grad(self, set_to_none: bool = True):
        if not self.fused:
            return self._fallback.zero_grad(set_to_none=set_to_none)
        dirty = not self._grad_is_zero
        for p in self._order:
            p.grad = None
            dirty = dirty or getattr(p, "grad_accumulated", False)
            p.grad_accumulated = False
        if dirty:  # after step() the update kernel has already cleared the arena
            self.grad.zero_()
            self._grad_is_zero = True

    def mark_grad_dirty(self) -> None:
        self._grad_is_zero = False

    def state_dict(self):
        if not self.fused:
            return self._fallback.state_dict()
        return {"fused": True, "step": self._step, "master": self.master, "m": self.m, "v": self.v, "shard": tuple(self.shard),
                "shapes": [tuple(p.shape) for p in self._order], "offsets": list(self.offsets),
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, sd):
        if not self.fused:
            return self._fallback.load_state_dict(sd)
        if [tuple(s) for s in sd["shapes"]] != [tuple(p.shape) for p in self._order]:
            raise ValueError("optimizer state was saved for a different parameter layout")
        if tuple(sd.get("shard", (0, self.total))) != tuple(self.shard):
            raise ValueError("optimizer state was saved with a different data-parallel sharding")
        self._step = int(sd["step"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        lib = _lib.require()
        _lib.check_rc(lib.b200_cast_f32_bf16(self.master.data_ptr(), self.p16.data_ptr(), self.total, 1.0, _lib.stream_ptr()), "cast")
        for g, saved in zip(self.param_groups, sd["param_groups"]):
            g.update(saved)


def _pad(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN
