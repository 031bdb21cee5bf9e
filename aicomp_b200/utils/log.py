"""Rank-tagged structured logging.

Level comes from ``AICOMP_LOG`` (default WARNING; the reference hard-codes
``logging.basicConfig(level=ERROR)`` in every module and prints unconditionally,
e.g. opt_prime/opt_prime/opti_pri.py:35).  ``rank0_print`` is for the few
user-facing progress lines.
"""
from __future__ import annotations

import logging
import os
import sys

_configured = False


def _configure() -> None:
    global _configured
    if _configured:
        return
    level = getattr(logging, os.environ.get("AICOMP_LOG", "WARNING").upper(), logging.WARNING)
    rank = os.environ.get("RANK", "0")
    handler = logging.StreamHandler(sys.stderr)
    handler.setFormatter(logging.Formatter(f"[%(asctime)s r{rank} %(levelname).1s %(name)s] %(message)s", "%H:%M:%S"))
    root = logging.getLogger("aicomp_b200")
    root.setLevel(level)
    root.addHandler(handler)
    root.propagate = False
    _configured = True


def get_logger(name: str) -> logging.Logger:
    _configure()
    if not name.startswith("aicomp_b200"):
        name = "aicomp_b200." + name
    return logging.getLogger(name)


def rank0_print(*args, **kwargs) -> None:
    if os.environ.get("RANK", "0") == "0":
        print(*args, **kwargs, flush=True)
