"""Packed-token dataset indices (C++ builders) and the datasets that use them.

``build_sample_idx`` / ``build_blending_indices`` are the native helpers of this framework's library
(``ops/csrc/data_helpers.cpp``); NumPy implementations are kept as the test oracle and as a fallback when the
library is not built.  ``PackedTokenDataset`` serves ``(input_ids, labels)`` windows of ``seq_len`` tokens over a
shuffled concatenation of documents, ``BlendedDataset`` mixes datasets by weight.  Role of the reference's
``gpt-neox/megatron/data`` (helpers.cpp, gpt2_dataset.py, blendable_dataset.py).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np


def _lib():
    from ..ops import _lib as L
    lib = L.load()
    if lib is None or not hasattr(lib, "b200_build_sample_idx"):
        return None
    lib.b200_num_samples.restype = ctypes.c_longlong
    lib.b200_num_samples.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_int]
    lib.b200_build_sample_idx.restype = ctypes.c_int
    lib.b200_build_sample_idx.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                          ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int]
    lib.b200_build_blending_indices.restype = ctypes.c_int
    lib.b200_build_blending_indices.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong]
    return lib


def num_samples(num_epochs: int, tokens_per_epoch: int, seq_len: int) -> int:
    return (num_epochs * tokens_per_epoch - 1) // seq_len


def build_sample_idx_numpy(sizes: np.ndarray, doc_idx: np.ndarray, seq_len: int, n_samples: int) -> np.ndarray:
    start = np.concatenate([[0], np.cumsum(sizes[doc_idx].astype(np.int64))])
    pos = np.arange(n_samples + 1, dtype=np.int64) * seq_len
    j = np.searchsorted(start[:-1], pos, side="right") - 1
    return np.stack([j, pos - start[j]], 1)


def build_sample_idx(sizes: np.ndarray, doc_idx: np.ndarray, seq_len: int, num_epochs: int, tokens_per_epoch: int,
                     threads: int = 8) -> np.ndarray:
    """``[num_samples + 1, 2]`` int64: for every sample boundary the position in ``doc_idx`` and the offset in that document."""
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
    n = num_samples(num_epochs, tokens_per_epoch, seq_len)
    lib = _lib()
    if lib is None:
        return build_sample_idx_numpy(sizes, doc_idx, seq_len, n)
    out = np.empty((n + 1, 2), dtype=np.int64)
    rc = lib.b200_build_sample_idx(sizes.ctypes.data, len(sizes), doc_idx.ctypes.data, len(doc_idx), seq_len, n, out.ctypes.data, threads)
    if rc:
        raise ValueError(f"build_sample_idx failed with code {rc}")
    return out


def build_blending_indices(weights: Sequence[float], size: int) -> Tuple[np.ndarray, np.ndarray]:
    w = np.ascontiguousarray(np.asarray(weights, dtype=np.float64) / np.sum(weights))
    ds = np.empty(size, dtype=np.uint8)
    si = np.empty(size, dtype=np.int64)
    lib = _lib()
    if lib is None:
        taken = np.zeros(len(w), dtype=np.int64)
        for i in range(size):
            d = int(np.argmax(w * max(i, 1) - taken))
            ds[i], si[i] = d, taken[d]
            taken[d] += 1
        return ds, si
    rc = lib.b200_build_blending_indices(ds.ctypes.data, si.ctypes.data, w.ctypes.data, len(w), size)
    if rc:
        raise ValueError(f"build_blending_indices failed with code {rc}")
    return ds, si


class PackedTokenDataset:
    """Windows of ``seq_len + 1`` tokens over shuffled, concatenated documents -> (input_ids, labels)."""

    def __init__(self, documents: List[np.ndarray], seq_len: int, num_epochs: int = 1, seed: int = 1234):
        self.docs = [np.asarray(d, dtype=np.int64) for d in documents]
        self.seq_len = seq_len
        sizes = np.array([len(d) for d in self.docs], dtype=np.int32)
        rng = np.random.RandomState(seed)
        self.doc_idx = np.concatenate([rng.permutation(len(self.docs)) for _ in range(num_epochs)]).astype(np.int32)
        self.sample_idx = build_sample_idx(sizes, self.doc_idx, seq_len, num_epochs, int(sizes.sum()))
        self.shuffle = rng.permutation(len(self.sample_idx) - 1)

    def __len__(self) -> int:
        return len(self.sample_idx) - 1

    def __getitem__(self, i: int):
        import torch
        i = int(self.shuffle[i])
        (j0, o0), (j1, o1) = self.sample_idx[i], self.sample_idx[i + 1]
        if j0 == j1:
            toks = self.docs[self.doc_idx[j0]][o0:o1 + 1]
        else:
            parts = [self.docs[self.doc_idx[j0]][o0:]]
            parts += [self.docs[self.doc_idx[j]] for j in range(j0 + 1, j1)]
            parts.append(self.docs[self.doc_idx[j1]][:o1 + 1])
            toks = np.concatenate(parts)
        t = torch.from_numpy(np.ascontiguousarray(toks[: self.seq_len + 1]))
        return t[:-1], t[1:]


class BlendedDataset:
    def __init__(self, datasets: List, weights: Sequence[float], size: Optional[int] = None):
        self.datasets = datasets
        self.size = size or sum(len(d) for d in datasets)
        self.ds_index, self.sample_index = build_blending_indices(weights, self.size)

    def __len__(self) -> int:
        return self.size

    def __getitem__(self, i: int):
        d = self.datasets[int(self.ds_index[i])]
        return d[int(self.sample_index[i]) % len(d)]
