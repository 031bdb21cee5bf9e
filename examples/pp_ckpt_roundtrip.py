"""Checkpoint round trips of a pipeline-parallel Llama on synthetic tokens.

    torchrun --nproc-per-node 2 examples/pp_ckpt_roundtrip.py --cpu --workdir /tmp/ckpt_demo

1. train a few steps, ``save_ckpt`` (native per-stage format with optimizer state), train on, then ``load_ckpt`` into
   a fresh engine and check that it continues with the same losses
   (opt_prime/examples/pp_train_gpt2_ckpt_save.py:137, pp_train_gpt2_ckpt_load.py:138-149);
2. ``save_hf_ckpt`` (``stage{S}_tp{T}.pt`` files) and merge them on rank 0 into a HuggingFace model directory that
   ``from_pretrained`` loads (opt_prime/examples/pp_train_llama_into_hf_ckpt.py, merge_hf_ckpt.py).
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from opt_prime.opti_pri import Optimus_p  # noqa: E402


def build():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(num_hidden_layers=4, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, intermediate_size=512,
                      vocab_size=1024, max_position_embeddings=256, tie_word_embeddings=False)
    torch.manual_seed(0)
    return cfg, LlamaForCausalLM(cfg)


def train_steps(engine, optimizer, steps, start, vocab):
    losses = []
    for step in range(start, start + steps):
        g = torch.Generator().manual_seed(100 + step)
        tokens = torch.randint(0, vocab, (8, 65), generator=g)
        labels = engine.move_labels2last_stage(tokens[:, 1:])
        optimizer.zero_grad()
        engine.run(tokens[:, :-1] if engine.is_first_stage() else None, labels, mode="1f1b")
        optimizer.step()
        loss = engine.get_loss()
        losses.append(sum(loss) / len(loss) if loss else None)
    return losses


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--workdir", default="ckpt_demo")
    a = ap.parse_args()
    os.makedirs(a.workdir, exist_ok=True)
    os.chdir(a.workdir)
    cfg, model = build()
    engine = Optimus_p(model, num_mb=4, use_gpu=not a.cpu, checkpoint=True, ckpt_dir_postfix="demo")
    optimizer = torch.optim.AdamW(engine.parameters(), lr=1e-3)
    engine.optimizer = optimizer
    train_steps(engine, optimizer, 3, 0, cfg.vocab_size)
    engine.save_ckpt(step=3, epoch=0)
    want = train_steps(engine, optimizer, 2, 3, cfg.vocab_size)          # what the uninterrupted run does next

    _, model2 = build()
    resumed = Optimus_p(model2, num_mb=4, use_gpu=not a.cpu, checkpoint=True, ckpt_dir_postfix="demo")
    opt2 = torch.optim.AdamW(resumed.parameters(), lr=1e-3)
    resumed.optimizer = opt2
    resumed.load_ckpt(step=3, epoch=0)
    got = train_steps(resumed, opt2, 2, 3, cfg.vocab_size)
    if engine.is_last_stage():
        print(f"resume: uninterrupted {[round(x, 5) for x in want]} vs resumed {[round(x, 5) for x in got]}")
        assert all(abs(x - y) < 1e-4 for x, y in zip(want, got)), "resumed run diverged"

    resumed.save_hf_ckpt("hf_stage_files", step=5, epoch=0)
    resumed.comm.barrier()
    if resumed.get_rank() == 0:
        from aicomp_b200.ckpt.merge_hf_ckpt import merge
        hf = merge(cfg, "hf_stage_files", output="merged_hf_model")
        print(f"merged HuggingFace model written to {os.path.abspath('merged_hf_model')} ({sum(p.numel() for p in hf.parameters())} parameters)")
    resumed.comm.barrier()


if __name__ == "__main__":
    main()
