"""Profile database: measured per-node times, ``known_cost/{model}_{gpu}_{tp}.npz``.

File format of the reference (fasop/README.md:74-86): key ``data``, shape ``(n_mbs, 10)``, milliseconds, rows for
micro-batch sizes 1, 2, 4, ...; columns in ``NODE_TYPES`` order.  The reference stores forward times only and
multiplies by 3.0 for forward+backward (fasop/config.py:725,843); files written by this framework also carry
``data_bwd`` with measured backward times, which is used when present.  When no file exists for a model/GPU an
analytic roofline estimate (FLOPs / sustained tensor throughput, bytes / HBM bandwidth) stands in.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import numpy as np

from .config import GPU_SPECS, MBS_OPTIONS, NODE_TYPES, ModelConfig

FWD_BWD_FACTOR = 3.0
HERE = os.path.dirname(os.path.abspath(__file__))


class ProfileDB:
    def __init__(self, model: ModelConfig, gpu: str, root: Optional[str] = None):
        self.model, self.gpu = model, gpu
        self.root = root or os.path.join(HERE, "known_cost")
        self._tables: Dict[int, Tuple[np.ndarray, Optional[np.ndarray]]] = {}
        self.sources: Dict[int, str] = {}

    def _load(self, tp: int):
        if tp in self._tables:
            return self._tables[tp]
        path = os.path.join(self.root, f"{self.model.name}_{self.gpu}_{tp}.npz")
        if os.path.exists(path):
            z = np.load(path)
            fwd = np.asarray(z["data"], dtype=np.float64)
            bwd = np.asarray(z["data_bwd"], dtype=np.float64) if "data_bwd" in z.files else None
            self.sources[tp] = path
        else:
            fwd, bwd = self._analytic(tp)
            self.sources[tp] = "analytic roofline"
        self._tables[tp] = (fwd, bwd)
        return fwd, bwd

    def _analytic(self, tp: int):
        spec = GPU_SPECS[self.gpu]
        m = self.model
        rows_f, rows_b = [], []
        for mbs in MBS_OPTIONS:
            T = mbs * m.seq_len
            f, b = [], []
            for node in NODE_TYPES:
                params = m.node_params_sharded(node, tp) if node != "embed" else 0
                flops = 2.0 * T * params
                if node == "attn_o":  # causal attention is charged here (as the reference's attribution does)
                    flops += 2.0 * 2.0 * T * m.seq_len * m.heads * m.head_dim / tp / 2
                bytes_ = 2.0 * T * m.node_act_elems(node, tp) * 2 + 2.0 * params
                t = max(flops / (0.75 * spec["bf16_flops"]), bytes_ / (0.8 * spec["hbm"])) + 6e-6
                f.append(t * 1e3)
                b.append(2.0 * t * 1e3)
            rows_f.append(f)
            rows_b.append(b)
        return np.array(rows_f), np.array(rows_b)

    def node_times(self, tp: int, mbs: int) -> Tuple[np.ndarray, np.ndarray]:
        """(forward, backward) seconds per node type for this tp and micro-batch size."""
        fwd, bwd = self._load(tp)
        row = MBS_OPTIONS.index(mbs) if mbs in MBS_OPTIONS else None
        if row is None or row >= fwd.shape[0]:
            # scale the largest measured row linearly
            last = fwd.shape[0] - 1
            k = mbs / MBS_OPTIONS[last]
            f = fwd[last] * k
            b = (bwd[last] * k) if bwd is not None else f * (FWD_BWD_FACTOR - 1.0)
        else:
            f = fwd[row]
            b = bwd[row] if bwd is not None else f * (FWD_BWD_FACTOR - 1.0)
        return f * 1e-3, b * 1e-3


def save_profile(path: str, fwd_ms: np.ndarray, bwd_ms: Optional[np.ndarray] = None) -> None:
    if bwd_ms is not None:
        np.savez(path, data=fwd_ms, data_bwd=bwd_ms)
    else:
        np.savez(path, data=fwd_ms)
