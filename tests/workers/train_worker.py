"""Rank body: trains a tiny model through Optimus_p and reports losses and a parameter checksum."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from tests.dist_utils import worker_args, worker_report  # noqa: E402
from tests.models_small import build_model, make_batch  # noqa: E402

from aicomp_b200 import Optimus_p  # noqa: E402


def main():
    a = worker_args()
    torch.manual_seed(0)
    model = build_model(a["model"])
    use_gpu = bool(a.get("use_gpu", False))
    e = Optimus_p(model, num_mb=a.get("num_mb", 2), use_gpu=use_gpu, pp_size=a.get("pp", 1), dp_size=a.get("dp", 1),
                  tp_size=a.get("tp", 1), activation_ckpt=a.get("act_ckpt", False), partitioner=a.get("partitioner", "auto"),
                  dtype=getattr(torch, a["dtype"]) if a.get("dtype") else None, sequence_parallel=a.get("sp", True),
                  dp_backend=a.get("dp_backend", "nccl"), tp_backend=a.get("tp_backend", "nccl"),
                  ir_analyze=__import__("aicomp_b200").IR_Anal[a.get("ir", "PARALLEL")], dynamo_capture=a.get("dynamo", False),
                  fused_kernels=False if a.get("dynamo") else None, cuda_graphs=a.get("graphs", False),
                  pp_backend=a.get("pp_backend", "auto"))
    if a.get("fused_adamw"):
        from aicomp_b200 import FusedAdamW
        opt = FusedAdamW(e.parameters(), lr=a.get("lr", 1e-3), grad_scale=1.0 / a.get("num_mb", 2), max_grad_norm=1.0,
                         norm_groups={"pp": e.tpl.pp_group} if e.tpl.pp_size > 1 else None)
        if e.dp is not None:
            opt.attach_to_reducer(e.dp, shard_state=a.get("shard", True))
    else:
        opt = torch.optim.AdamW(e.parameters(), lr=a.get("lr", 1e-3))
    e.optimizer = opt
    losses = []
    for step in range(a.get("steps", 3)):
        ids, labels = make_batch(a["model"], a.get("batch", 4), seed=step, seq=a.get("seq", 16))
        if e.tpl.dp_size > 1:  # each replica takes its slice of the global batch
            per = ids.shape[0] // e.tpl.dp_size
            sl = slice(e.tpl.dp_rank * per, (e.tpl.dp_rank + 1) * per)
            ids, labels = ids[sl], labels[sl]
        lab = e.move_labels2last_stage(labels)
        opt.zero_grad()
        e.run(ids if e.is_first_stage() else None, lab, mode=a.get("mode", "1f1b"))
        if a.get("clip"):
            e.clip_grad_norm_(a["clip"])
        opt.step()
        l = e.get_loss()
        losses.append(sum(l) / len(l) if l is not None else None)
    checksum = float(sum(p.detach().double().abs().sum().item() for p in e.parameters()))
    worker_report({"losses": losses, "pp_backend": getattr(e, "pp_backend", None), "graphs": bool(e.cuda_graphs and e._graphed), "stage": e.tpl.stage, "dp_rank": e.tpl.dp_rank, "tp_rank": e.tpl.tp_rank,
                   "checksum": checksum, "n_params": sum(p.numel() for p in e.parameters())})
    e.comm.barrier()


if __name__ == "__main__":
    main()
