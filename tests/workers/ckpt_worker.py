"""Rank body: train a few steps, write checkpoints, optionally resume."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from tests.dist_utils import worker_args, worker_report  # noqa: E402
from tests.models_small import build_model, make_batch  # noqa: E402

from aicomp_b200 import Optimus_p  # noqa: E402


def train(e, opt, steps, start=0):
    losses = []
    for step in range(start, start + steps):
        ids, labels = make_batch("llama", 4, seed=step)
        lab = e.move_labels2last_stage(labels)
        opt.zero_grad()
        e.run(ids if e.is_first_stage() else None, lab, mode="1f1b")
        opt.step()
        l = e.get_loss()
        losses.append(sum(l) / len(l) if l else None)
    return losses


def main():
    a = worker_args()
    os.chdir(a["dir"]) if os.path.isdir(a["dir"]) else (os.makedirs(a["dir"], exist_ok=True), os.chdir(a["dir"]))
    torch.manual_seed(0)
    e = Optimus_p(build_model("llama"), num_mb=2, use_gpu=False, pp_size=a["pp"], tp_size=a["tp"], checkpoint=True,
                  ckpt_dir_postfix="t", tp_backend="nccl")
    opt = torch.optim.AdamW(e.parameters(), lr=1e-3)
    e.optimizer = opt
    out = {"losses": [None]}
    mode = a.get("native")
    if mode == "straight":
        out["losses"] = train(e, opt, 4)
    elif mode == "resume":
        l1 = train(e, opt, 2)
        e.save_ckpt(step=2, epoch=0)
        e.comm.barrier()
        # a fresh engine state: scramble weights, then restore
        with torch.no_grad():
            for p in e.parameters():
                p.add_(1.0)
        e.load_ckpt(step=2, epoch=0)
        out["losses"] = l1 + train(e, opt, 2, start=2)
    else:
        train(e, opt, 2)
        e.save_hf_ckpt(os.path.join(a["dir"], "hf"), step=2, epoch=0)
        # probe: logits checksum through the pipeline on a fixed batch
        e.eval()
        e.preserve_output = True
        ids, _ = make_batch("llama", 2, seed=99)
        e.run(ids if e.is_first_stage() else None, None, mode="gpipe")
        if e.is_last_stage():
            logits = torch.cat([o["logits"] for o in e.outputs])
            out["probe"] = float(logits.double().abs().sum())
    worker_report(out)
    e.comm.barrier()


if __name__ == "__main__":
    main()
