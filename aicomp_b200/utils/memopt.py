"""Memory relief around a training step: cache trimming and optimizer/model offload to host (or disk).

Capability of the reference's "mopt" code (opt_prime/opt_prime/schedule.py:222-443, 927-955): when free
device memory drops under a threshold, release the caching allocator's unused blocks; optionally keep
the optimizer state on the host during forward/backward (``swap_opt_in_fwdbwd``) and move parameters and
gradients to the host so that ``optimizer.step()`` runs there (``swap_model_in_optstep``), optionally
spilling optimizer state to a per-rank file (``swap_use_disk``).  Thresholds are the reference's 4 / 5 /
25 GB (opti_pri.py:682-685).  On a 180 GB B200 these paths are rarely needed; they are kept for parity.
"""
from __future__ import annotations

import gc
import os

import torch

FREE_MEM_GC_BYTES = 4 << 30
FREE_MEM_OFFLOAD_OPT_BYTES = 5 << 30
FREE_MEM_OFFLOAD_MODEL_BYTES = 25 << 30


def free_device_bytes(device: torch.device) -> int:
    if device.type != "cuda":
        return 1 << 62
    total = torch.cuda.get_device_properties(device).total_memory
    return total - torch.cuda.memory_reserved(device)


def cond_free_mem(engine) -> None:
    if engine.device.type == "cuda" and (engine.force_free_mem or free_device_bytes(engine.device) < FREE_MEM_GC_BYTES):
        gc.collect()
        torch.cuda.empty_cache()


def _state_tensors(optimizer):
    for st in optimizer.state.values():
        for k, v in st.items():
            if isinstance(v, torch.Tensor):
                yield st, k, v


def offload_optimizer(engine) -> None:
    opt = engine.optimizer
    if opt is None or getattr(engine, "_opt_offloaded", False):
        return
    if engine.swap_use_disk:
        path = f"temp_optistat_{engine.comm.rank}"
        torch.save({i: {k: v.cpu() for k, v in st.items() if isinstance(v, torch.Tensor)} for i, st in enumerate(opt.state.values())}, path)
        for st, k, v in list(_state_tensors(opt)):
            st[k] = torch.empty(0, dtype=v.dtype)
            st.setdefault("_shape_" + k, tuple(v.shape))
        engine._opt_disk = path
    else:
        for st, k, v in list(_state_tensors(opt)):
            st[k] = v.to("cpu", non_blocking=True)
    engine._opt_offloaded = True


def load_optimizer(engine) -> None:
    opt = engine.optimizer
    if opt is None or not getattr(engine, "_opt_offloaded", False):
        return
    if getattr(engine, "_opt_disk", None):
        saved = torch.load(engine._opt_disk)
        for i, st in enumerate(opt.state.values()):
            for k, v in saved[i].items():
                st[k] = v.to(engine.device)
        os.remove(engine._opt_disk)
        engine._opt_disk = None
    else:
        for st, k, v in list(_state_tensors(opt)):
            st[k] = v.to(engine.device, non_blocking=True)
    engine._opt_offloaded = False


def offload_model(engine) -> None:
    """Move parameters and gradients to the host so the optimizer steps there."""
    if getattr(engine, "_model_offloaded", False):
        return
    for p in engine.stage_module.parameters():
        g = p.grad
        p.data = p.data.to("cpu")
        if g is not None:
            p.grad = g.to("cpu")
    if engine.optimizer is not None:
        for st, k, v in list(_state_tensors(engine.optimizer)):
            st[k] = v.to("cpu")
    engine._model_offloaded = True


def load_model(engine) -> None:
    if not getattr(engine, "_model_offloaded", False):
        return
    for p in engine.stage_module.parameters():
        g = p.grad
        p.data = p.data.to(engine.device)
        if g is not None:
            p.grad = g.to(engine.device)
    if engine.optimizer is not None and not engine.swap_opt_in_fwdbwd:
        for st, k, v in list(_state_tensors(engine.optimizer)):
            st[k] = v.to(engine.device)
    engine._model_offloaded = False


def before_run(engine) -> None:
    if engine.device.type != "cuda":
        return
    cond_free_mem(engine)
    if engine.swap_model_in_optstep:
        load_model(engine)
    if engine.swap_opt_in_fwdbwd and (engine.force_free_mem or free_device_bytes(engine.device) < FREE_MEM_OFFLOAD_OPT_BYTES):
        offload_optimizer(engine)


def after_run(engine) -> None:
    if engine.device.type != "cuda":
        return
    if engine.swap_model_in_optstep and engine.training and \
            (engine.force_free_mem or free_device_bytes(engine.device) < FREE_MEM_OFFLOAD_MODEL_BYTES):
        offload_model(engine)
    elif engine.swap_opt_in_fwdbwd:
        load_optimizer(engine)
    if engine.display_mem:
        print(f"[rank {engine.comm.rank}] allocated {torch.cuda.memory_allocated() / 2**30:.2f} GiB, "
              f"reserved {torch.cuda.memory_reserved() / 2**30:.2f} GiB")
