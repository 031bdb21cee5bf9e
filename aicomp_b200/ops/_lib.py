"""ctypes binding of the in-tree sm_100a kernel library.

The library is built by :mod:`aicomp_b200.ops.build`.  On a machine with a GPU a
missing or unloadable library is an error (ops never fall back silently there);
without a GPU the Python reference implementations in :mod:`aicomp_b200.ops`
are used and the library is not needed.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build as _build

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_load_error: Optional[str] = None

P = c_void_p
I = c_int
L = c_longlong
F = c_float

_PROTOS = {
    "b200_gemm_bf16": [P, P, P, P, I, I, I, L, L, L, I, I, I, F, I, I, I, P, P],
    "b200_gemm2_bf16": [P, P, P, P, I, I, I, L, L, L, I, I, I, F, I, P, P],
    "b200_gemm2_supported": [I, I, I],
    "b200_norm_bwd_ctas": [],
    "b200_norm_fwd": [P, P, P, P, P, P, P, P, I, I, F, I, P],
    "b200_norm_bwd": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P],
    "b200_rope": [P, P, P, P, L, I, I, L, F, P],
    "b200_swiglu_fwd": [P, P, L, I, P],
    "b200_swiglu_bwd": [P, P, P, L, I, P],
    "b200_gelu_fwd": [P, P, L, P],
    "b200_gelu_bwd": [P, P, P, L, P],
    "b200_cross_entropy": [P, P, P, L, I, L, I, F, P, I, P],
    "b200_embedding_fwd": [P, P, P, L, I, I, P],
    "b200_embedding_bwd": [P, P, P, L, I, I, P],
    "b200_softmax_fwd": [P, P, P, L, I, I, F, I, I, I, P],
    "b200_softmax_bwd": [P, P, P, L, I, F, P],
    "b200_adamw": [P, P, P, P, P, P, P, L, F, F, F, F, F, I, F, F, I, P],
    "b200_sumsq": [P, L, P, P],
    "b200_cast_f32_bf16": [P, P, L, F, P],
    "b200_accum_bf16_f32": [P, P, L, P],
}

# Entry points added by later kernels register here (name -> argtypes).
OPTIONAL_PROTOS = {}


def _bind(lib: ctypes.CDLL) -> None:
    for name, argtypes in list(_PROTOS.items()) + list(OPTIONAL_PROTOS.items()):
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if name in _PROTOS:
                raise
            continue
        fn.argtypes = argtypes
        fn.restype = c_int


def rebind() -> None:
    """Bind entry points registered in ``OPTIONAL_PROTOS`` after the library was loaded."""
    if _lib is not None:
        _bind(_lib)


def load(required: bool = False) -> Optional[ctypes.CDLL]:
    """Load (building first if the sources changed and nvcc is present)."""
    global _lib, _load_error
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            path = _build.lib_path()
            if not _build.is_current():
                try:
                    path = _build.build()
                except Exception as e:  # no nvcc on this machine: use a prebuilt library if there is one
                    if not path.exists():
                        raise RuntimeError(f"kernel library missing and cannot be built: {e}") from e
            lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
            _bind(lib)
            _lib = lib
        except Exception as e:
            _load_error = repr(e)
            if required:
                raise
            return None
    return _lib


def have_gpu_kernels() -> bool:
    """True when CUDA tensors will be served by the sm_100a kernels."""
    return torch.cuda.is_available() and load() is not None


def require() -> ctypes.CDLL:
    lib = load(required=True)
    assert lib is not None
    return lib


def load_error() -> Optional[str]:
    return _load_error


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


# --- per-device error word written by bounded waits inside kernels ----------
_err_words = {}


def err_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _err_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _err_words[idx] = w
    return w


_ERR_NAMES = {1: "consumer wait for TMA stage", 2: "producer wait for free stage", 3: "epilogue wait for accumulator",
              4: "MMA wait for drained accumulator", 5: "wait for a peer GPU's flag", 6: "bad argument",
              7: "dynamic shared memory window not 1024-byte aligned"}


def check_errors(device: Optional[torch.device] = None) -> None:
    """Synchronising check of the kernel status word; raises if a bounded wait ran out."""
    for idx, w in list(_err_words.items()):
        if device is not None and device.index not in (None, idx):
            continue
        code = int(w.item())
        if code != 0:
            w.zero_()
            raise RuntimeError(f"sm_100a kernel reported error {code} ({_ERR_NAMES.get(code, 'unknown')}) on cuda:{idx}")


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: kernel launcher returned {rc}")
