"""Metrics sink: JSON-lines records of step time (max over ranks), throughput, loss, memory, bytes moved.

The reference prints wall-clock ``ms/batch`` from its examples and logs TensorBoard scalars in the demo scripts
(opt_prime/demo/pp_train_llama-8b.py:117-121,198-209).  ``MetricsLogger`` writes one JSON object per step on rank
0, optionally mirrors scalars to TensorBoard when it is installed, and ``StepTimer`` measures steps with CUDA
events on the launching stream.
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist


class StepTimer:
    """CUDA-event timer around a step; ``elapsed_ms(max_over_ranks=True)`` reduces with MAX over the world."""

    def __init__(self, device: Optional[torch.device] = None):
        self.device = device
        self.cuda = device is not None and device.type == "cuda"
        if self.cuda:
            self._s, self._e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._t0 = 0.0
        self._ms = 0.0

    def start(self) -> None:
        if self.cuda:
            self._s.record()
        self._t0 = time.perf_counter()

    def stop(self) -> None:
        if self.cuda:
            self._e.record()
        else:
            self._ms = (time.perf_counter() - self._t0) * 1e3

    def elapsed_ms(self, max_over_ranks: bool = True, group=None) -> float:
        if self.cuda:
            self._e.synchronize()
            ms = self._s.elapsed_time(self._e)
        else:
            ms = self._ms
        if max_over_ranks and dist.is_available() and dist.is_initialized():
            t = torch.tensor([ms], dtype=torch.float64, device=self.device if self.cuda else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            ms = float(t.item())
        return ms


class MetricsLogger:
    def __init__(self, path: Optional[str] = None, rank: int = 0, tensorboard_dir: Optional[str] = None):
        self.rank = rank
        self.path = path
        self._f = open(path, "a") if (path and rank == 0) else None
        self._tb = None
        if tensorboard_dir and rank == 0:
            try:
                from torch.utils.tensorboard import SummaryWriter
                self._tb = SummaryWriter(tensorboard_dir)
            except Exception:
                self._tb = None

    def log(self, step: int, **values: Any) -> Dict[str, Any]:
        rec = {"step": step, "time": time.time(), **values}
        if self._f:
            self._f.write(json.dumps(rec) + "\n")
            self._f.flush()
        if self._tb:
            for k, v in values.items():
                if isinstance(v, (int, float)):
                    self._tb.add_scalar(k, v, step)
        return rec

    def log_train_step(self, step: int, step_ms: float, tokens: int, loss: Optional[float] = None, device=None, **extra):
        vals = {"Train/ms_per_batch": step_ms, "Train/tokens_per_s": tokens / (step_ms / 1e3) if step_ms > 0 else 0.0}
        if loss is not None:
            vals["Train/Loss"] = loss
            vals["Train/Perplexity"] = float(torch.exp(torch.tensor(min(loss, 50.0))))
        if device is not None and torch.device(device).type == "cuda":
            vals["mem/allocated_gib"] = torch.cuda.memory_allocated(device) / 2**30
            vals["mem/reserved_gib"] = torch.cuda.memory_reserved(device) / 2**30
        vals.update(extra)
        return self.log(step, **vals)

    def close(self) -> None:
        if self._f:
            self._f.close()
        if self._tb:
            self._tb.close()
