"""LoRA fine-tuning under pipeline/tensor parallelism, then merge and save an HF-compatible checkpoint."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from opt_prime.lora import LoRAConfig  # noqa: E402
from opt_prime.opti_pri import Optimus_p  # noqa: E402


def main():
    from transformers import LlamaConfig, LlamaForCausalLM
    cpu = "--cpu" in sys.argv
    cfg = LlamaConfig(num_hidden_layers=4, hidden_size=512, num_attention_heads=4, num_key_value_heads=2, intermediate_size=1024,
                      vocab_size=8192, max_position_embeddings=1024, tie_word_embeddings=False)
    torch.manual_seed(0)
    eng = Optimus_p(LlamaForCausalLM(cfg), num_mb=2, use_gpu=not cpu, dtype=None if cpu else torch.bfloat16)
    n = eng.apply_lora(LoRAConfig(r=8, alpha=16, dropout=0.05))
    opt = torch.optim.AdamW(eng.parameters(), lr=1e-3)
    print(f"rank {eng.get_rank()}: {n} adapted projections, {sum(p.numel() for p in eng.parameters())} trainable parameters")
    g = torch.Generator().manual_seed(0)
    for step in range(10):
        tokens = torch.randint(0, cfg.vocab_size, (4, 257), generator=g)
        labels = eng.move_labels2last_stage(tokens[:, 1:])
        opt.zero_grad()
        eng.run(tokens[:, :-1] if eng.is_first_stage() else None, labels, mode="1f1b")
        opt.step()
        if eng.is_last_stage():
            print(f"step {step}: loss {sum(eng.get_loss()) / 2:.4f}")
    eng.save_lora_ckpt(step=10, epoch=0)
    eng.merge_lora()
    eng.save_hf_ckpt("lora_merged_hf", step=10, epoch=0)


if __name__ == "__main__":
    main()
