"""Pipeline-parallel GPT-2 training (synthetic tokens).  CPU/gloo: ``torchrun --nproc-per-node 2 examples/pp_train_gpt2.py --cpu``.

Mirrors the canonical user loop of the reference (opt_prime/examples/pp_train_gpt2.py:88-133): shift labels, move
them to the last stage, zero_grad, run the 1F1B (or GPipe) schedule, read the loss on the last stage, clip, step.
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from opt_prime.opti_pri import Optimus_p  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--mode", default="gpipe", choices=["gpipe", "1f1b"])
    ap.add_argument("--dynamo-capture", action="store_true")
    a = ap.parse_args()
    from transformers import GPT2Config, GPT2LMHeadModel
    torch.manual_seed(0)
    cfg = GPT2Config(n_layer=12, n_embd=768, n_head=12, vocab_size=50257, n_positions=128, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    model = GPT2LMHeadModel(cfg)
    for p in model.parameters():
        torch.nn.init.normal_(p, 0.0, 0.02) if p.dim() > 1 else None
    engine = Optimus_p(model, num_mb=4, use_gpu=not a.cpu, dynamo_capture=a.dynamo_capture)
    engine.train()
    optimizer = torch.optim.AdamW(engine.parameters(), lr=1e-4)
    engine.optimizer = optimizer
    g = torch.Generator().manual_seed(0)
    for step in range(a.steps):
        tokens = torch.randint(0, cfg.vocab_size, (8, 129), generator=g)
        data, labels = tokens[:, :-1], tokens[:, 1:]
        t0 = time.time()
        labels = engine.move_labels2last_stage(labels)
        optimizer.zero_grad()
        engine.run(data if engine.is_first_stage() else None, labels, mode=a.mode)
        loss = engine.get_loss()
        torch.nn.utils.clip_grad_norm_(engine.parameters(), 0.5)
        optimizer.step()
        if engine.is_last_stage():
            print(f"step {step}: loss {sum(loss) / len(loss):.4f}  {1e3 * (time.time() - t0):.0f} ms/batch", flush=True)
    engine.comm.barrier()


if __name__ == "__main__":
    main()
