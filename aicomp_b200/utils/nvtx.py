"""NVTX ranges per (stage, micro-batch, F/B, send/recv), enabled with ``AICOMP_NVTX=1``.

The reference has no tracing in opt_prime; its MLPerf fork gates NVTX by
environment (mlperf/pytorch-22.09/scaleoutbridge.py:49-121).
"""
from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("AICOMP_NVTX", "0") == "1" and torch.cuda.is_available()


@contextlib.contextmanager
def range(name: str):  # noqa: A001 - mirrors torch.cuda.nvtx.range
    if _ENABLED:
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield
