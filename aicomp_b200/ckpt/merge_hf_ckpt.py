"""Merge ``stage{S}_tp{T}.pt`` files into one HuggingFace model directory (CPU tool).

    python -m aicomp_b200.ckpt.merge_hf_ckpt --model <hf name or config dir> --ckpt-dir <dir> --output <dir> [--token T]

Role of the reference's ``examples/merge_hf_ckpt.py``: keys are restored to HF fully-qualified names
(files written by the reference use flattened names - ``moved_`` prefix, ``.`` replaced by ``_`` - which
are looked up in a table built from a meta-device instance of the model), tensor-parallel shards are
concatenated (q/k/v/gate/up along dim 0, o/down along dim 1), the result is loaded with ``strict=True``
and written with ``save_pretrained``.
"""
from __future__ import annotations

import argparse
import glob
import os
import re
from typing import Dict, List, Optional

import torch

COLWISE = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
ROWWISE = ("o_proj", "down_proj")


def tp_concat_dim(key: str) -> Optional[int]:
    if not key.endswith(".weight"):
        return None
    for n in COLWISE:
        if f".{n}." in key:
            return 0
    for n in ROWWISE:
        if f".{n}." in key:
            return 1
    return None


def restore_key(key: str, original: Dict[str, str]) -> Optional[str]:
    """Map a stored key to its HF name; ``original`` maps flattened names (dots -> underscores) to HF names."""
    if key in original.values():
        return key
    bare = key[len("moved_"):] if key.startswith("moved_") else key
    return original.get(bare.replace(".", "_"))


def merge_state_dicts(files: List[str], original_keys: List[str]) -> Dict[str, torch.Tensor]:
    flat = {k.replace(".", "_"): k for k in original_keys}
    shards: Dict[str, Dict[int, torch.Tensor]] = {}
    tp_size = 1
    for f in files:
        blob = torch.load(f, map_location="cpu", weights_only=False)
        tp_size = max(tp_size, int(blob.get("tp_size", 1)))
        for key, val in blob["state_dict"].items():
            hf = restore_key(key, flat)
            if hf is None:
                continue  # non-persistent buffers such as rotary inv_freq are rebuilt by the model
            shards.setdefault(hf, {})[int(blob.get("tp_rank", 0))] = val
    merged: Dict[str, torch.Tensor] = {}
    for key, parts in shards.items():
        dim = tp_concat_dim(key)
        if dim is None or len(parts) == 1:
            merged[key] = parts[min(parts)]
        else:
            if sorted(parts) != list(range(tp_size)):
                raise ValueError(f"{key}: tensor-parallel shards {sorted(parts)} incomplete for tp_size {tp_size}")
            merged[key] = torch.cat([parts[r] for r in range(tp_size)], dim=dim)
    return merged


def merge(model_name_or_cfg, ckpt_dir: str, output: Optional[str] = None, token: Optional[str] = None, dtype=None):
    """Returns the merged HF model (and writes it when ``output`` is given)."""
    from transformers import AutoConfig, AutoModelForCausalLM
    cfg = model_name_or_cfg if not isinstance(model_name_or_cfg, str) else AutoConfig.from_pretrained(model_name_or_cfg, token=token)
    with torch.device("meta"):
        skeleton = AutoModelForCausalLM.from_config(cfg)
    keys = list(skeleton.state_dict().keys())
    files = sorted(glob.glob(os.path.join(ckpt_dir, "stage*_tp*.pt")),
                   key=lambda f: tuple(map(int, re.findall(r"stage(\d+)_tp(\d+)", os.path.basename(f))[0])))
    if not files:
        raise FileNotFoundError(f"no stage*_tp*.pt files in {ckpt_dir}")
    sd = merge_state_dicts(files, keys)
    model = AutoModelForCausalLM.from_config(cfg)
    tied = getattr(cfg, "tie_word_embeddings", False)
    if tied and "lm_head.weight" not in sd and "model.embed_tokens.weight" in sd:
        sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
    if dtype is not None:
        sd = {k: v.to(dtype) if v.is_floating_point() else v for k, v in sd.items()}
        model = model.to(dtype)
    model.load_state_dict(sd, strict=True)
    if output:
        model.save_pretrained(output)
        if isinstance(model_name_or_cfg, str):
            try:
                from transformers import AutoTokenizer
                AutoTokenizer.from_pretrained(model_name_or_cfg, token=token).save_pretrained(output)
            except Exception:
                pass
    return model


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", required=True)
    ap.add_argument("--ckpt-dir", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--token", default=os.environ.get("LLAMA_ACCESS_TOKEN"))
    a = ap.parse_args()
    merge(a.model, a.ckpt_dir, a.output, a.token)
    print(f"merged checkpoint written to {a.output}")


if __name__ == "__main__":
    main()
