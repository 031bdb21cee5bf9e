"""Native per-stage training checkpoints.

File contract of the reference (opt_prime/opt_prime/opti_pri.py:1192-1226): a dict
``{epoch, stage, stage_state_dict, optimizer_state_dict}`` saved as
``checkpoint_<postfix>_<stage>/ckpt_step_<s>_epoch_<e>.pt``, newest two kept.  Differences, all
backwards compatible when reading:

* data-parallel replica 0 writes; tensor-parallel ranks > 0 add a ``_tp<r>`` suffix (the reference
  lets every replica overwrite the same path);
* writes are atomic (temp file + rename) and a ``step``/RNG record is added so a resumed run
  continues the same random stream;
* directories written with ``ckpt_dir_postfix=None`` are still found as ``checkpoint_None_<stage>``.
"""
from __future__ import annotations

import glob
import os
import re
from typing import Optional

import torch


def _path(engine, step: int, epoch: int) -> str:
    tp = engine.tpl.tp_rank
    suffix = f"_tp{tp}" if tp > 0 else ""
    return os.path.join(engine.ckpt_dir, f"ckpt_step_{step}_epoch_{epoch}{suffix}.pt")


def save_ckpt(engine, step: int, epoch: int, keep: int = 2) -> Optional[str]:
    if not engine.checkpoint:
        raise RuntimeError("construct the engine with checkpoint=True to save checkpoints")
    sharded_opt = engine.optimizer is not None and getattr(engine.optimizer, "_dp_group", None) is not None
    if engine.tpl.dp_rank != 0:
        if sharded_opt:  # every data-parallel rank owns a slice of the optimizer state
            if engine.use_gpu:
                torch.cuda.synchronize()
            os.makedirs(engine.ckpt_dir, exist_ok=True)
            shard_path = _path(engine, step, epoch) + f".optdp{engine.tpl.dp_rank}"
            torch.save({"optimizer_state_dict": _cpu_tree(engine.optimizer.state_dict())}, shard_path + ".tmp")
            os.replace(shard_path + ".tmp", shard_path)
            return shard_path
        return None
    if engine.use_gpu:
        torch.cuda.synchronize()
    os.makedirs(engine.ckpt_dir, exist_ok=True)
    path = _path(engine, step, epoch)
    state = {
        "epoch": epoch, "step": step, "stage": engine.tpl.stage,
        "stage_state_dict": {k: v.detach().cpu() for k, v in engine.stage_module.state_dict().items()},
        "optimizer_state_dict": _cpu_tree(engine.optimizer.state_dict()) if engine.optimizer is not None else None,
        "rng_state": torch.get_rng_state(),
        "cuda_rng_state": torch.cuda.get_rng_state() if engine.use_gpu else None,
        "layout": {"pp": engine.tpl.pp_size, "dp": engine.tpl.dp_size, "tp": engine.tpl.tp_size},
    }
    tmp = path + ".tmp"
    torch.save(state, tmp)
    os.replace(tmp, path)
    _prune(engine, keep)
    return path


def _cpu_tree(x):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu()
    if isinstance(x, dict):
        return {k: _cpu_tree(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_cpu_tree(v) for v in x)
    return x


def _prune(engine, keep: int) -> None:
    tp = engine.tpl.tp_rank
    suffix = f"_tp{tp}" if tp > 0 else ""
    pat = re.compile(r"ckpt_step_(\d+)_epoch_(\d+)" + re.escape(suffix) + r"\.pt$")
    found = []
    for f in glob.glob(os.path.join(engine.ckpt_dir, "ckpt_step_*.pt")):
        m = pat.search(os.path.basename(f))
        if m:
            found.append(((int(m.group(2)), int(m.group(1))), f))
    found.sort()
    for _, f in found[:-keep] if keep > 0 else []:
        try:
            os.remove(f)
        except OSError:
            pass


def load_ckpt(engine, step: int, epoch: int) -> dict:
    if not engine.checkpoint:
        raise RuntimeError("construct the engine with checkpoint=True to load checkpoints")
    path = _path(engine, step, epoch)
    if not os.path.exists(path) and engine.tpl.tp_rank == 0:
        alt = os.path.join(f"checkpoint_None_{engine.tpl.stage}", os.path.basename(path))
        if os.path.exists(alt):
            path = alt
    state = torch.load(path, map_location="cpu", weights_only=False)
    if state.get("stage", engine.tpl.stage) != engine.tpl.stage:
        raise ValueError(f"checkpoint is for stage {state['stage']}, this rank runs stage {engine.tpl.stage}")
    engine.stage_module.load_state_dict(state["stage_state_dict"])
    opt_state = state.get("optimizer_state_dict")
    if engine.optimizer is not None and getattr(engine.optimizer, "_dp_group", None) is not None and engine.tpl.dp_rank != 0:
        opt_state = torch.load(path + f".optdp{engine.tpl.dp_rank}", map_location="cpu", weights_only=False)["optimizer_state_dict"]
    if engine.optimizer is not None and opt_state is not None:
        engine.optimizer.load_state_dict(opt_state)
    if state.get("rng_state") is not None:
        torch.set_rng_state(state["rng_state"])
    if engine.use_gpu and state.get("cuda_rng_state") is not None:
        torch.cuda.set_rng_state(state["cuda_rng_state"])
    return {"step": state.get("step", step), "epoch": state.get("epoch", epoch)}
