"""3D-parallel Llama training: ``torchrun --nproc-per-node 8 examples/pp_train_llama_3d.py --pp 2 --tp 2 --dp 2``.

bf16 weights with fp32 master weights / fused AdamW, 1F1B, fused tensor-parallel and data-parallel kernels.
Equivalent of the reference's ``pp_train_llama5.py`` family (pp/tp/dp combinations) on synthetic tokens.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aicomp_b200 import FusedAdamW, Optimus_p  # noqa: E402
from aicomp_b200.utils.metrics import MetricsLogger, StepTimer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    for k, d in (("pp", 1), ("tp", 1), ("dp", 1), ("layers", 8), ("hidden", 2048), ("seq", 2048), ("num-mb", 4), ("steps", 10)):
        ap.add_argument(f"--{k}", type=int, default=d)
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--save-hf", default=None, help="directory for stage*_tp*.pt files after training")
    a = ap.parse_args()
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(num_hidden_layers=a.layers, hidden_size=a.hidden, num_attention_heads=a.hidden // 128, num_key_value_heads=max(1, a.hidden // 512),
                      intermediate_size=int(3.5 * a.hidden), vocab_size=32000, max_position_embeddings=max(4096, a.seq), tie_word_embeddings=False)
    with torch.device("meta"):
        model = LlamaForCausalLM(cfg)
    eng = Optimus_p(model, num_mb=a.num_mb, use_gpu=not a.cpu, pp_size=a.pp, tp_size=a.tp, dp_size=a.dp,
                    dtype=None if a.cpu else torch.bfloat16)
    opt = FusedAdamW(eng.parameters(), lr=3e-4, grad_scale=1.0 / a.num_mb, max_grad_norm=1.0,
                     norm_groups={"pp": eng.tpl.pp_group, "tp": eng.tpl.tp_group})
    eng.optimizer = opt
    if eng.dp is not None:
        opt.attach_to_reducer(eng.dp)
    log = MetricsLogger("train_metrics.jsonl", rank=eng.get_rank())
    timer = StepTimer(eng.device)
    g = torch.Generator().manual_seed(eng.tpl.dp_rank)
    for step in range(a.steps):
        tokens = torch.randint(0, cfg.vocab_size, (a.num_mb, a.seq + 1), generator=g)
        timer.start()
        labels = eng.move_labels2last_stage(tokens[:, 1:])
        opt.zero_grad()
        eng.run(tokens[:, :-1] if eng.is_first_stage() else None, labels, mode="1f1b")
        opt.step()
        timer.stop()
        ms = timer.elapsed_ms()
        loss = eng.get_loss()
        if eng.is_last_stage() and eng.tpl.tp_rank == 0 and eng.tpl.dp_rank == 0:
            print(f"step {step}: loss {sum(loss) / len(loss):.4f}  {ms:.1f} ms", flush=True)
        log.log_train_step(step, ms, tokens=a.num_mb * a.seq * a.dp, loss=None if loss is None else sum(loss) / len(loss), device=eng.device)
    if a.save_hf:
        eng.save_hf_ckpt(a.save_hf, step=a.steps, epoch=0)
    eng.comm.barrier()


if __name__ == "__main__":
    main()
