"""Tiny deterministic models and batches shared by the CPU tests."""
import torch
import torch.nn as nn


def build_model(name: str):
    torch.manual_seed(0)
    if name == "gpt2":
        from transformers import GPT2Config, GPT2LMHeadModel
        cfg = GPT2Config(n_layer=4, n_embd=64, n_head=4, vocab_size=512, n_positions=64, resid_pdrop=0.0, embd_pdrop=0.0,
                         attn_pdrop=0.0, tie_word_embeddings=False)
        return GPT2LMHeadModel(cfg)
    if name == "llama":
        from transformers import LlamaConfig, LlamaForCausalLM
        cfg = LlamaConfig(num_hidden_layers=4, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                          vocab_size=512, max_position_embeddings=128, tie_word_embeddings=False)
        return LlamaForCausalLM(cfg)
    if name == "llama_d128":  # head_dim 128 and tile-sized widths: exercises the sm_100a attention / fused TP kernels
        from transformers import LlamaConfig, LlamaForCausalLM
        cfg = LlamaConfig(num_hidden_layers=2, hidden_size=512, num_attention_heads=4, num_key_value_heads=2, intermediate_size=1024,
                          vocab_size=512, max_position_embeddings=512, tie_word_embeddings=False)
        return LlamaForCausalLM(cfg)
    if name == "mlp":
        return nn.Sequential(*[m for _ in range(6) for m in (nn.Linear(32, 32), nn.ReLU())])
    raise ValueError(name)


def make_batch(name: str, batch: int, seed: int = 0, seq: int = 16):
    if name == "llama_d128" and seq == 16:
        seq = 256
    g = torch.Generator().manual_seed(1000 + seed)
    if name == "mlp":
        x = torch.randn(batch, 32, generator=g)
        return x, torch.randn(batch, 32, generator=g)
    ids = torch.randint(0, 512, (batch, seq), generator=g)
    labels = torch.cat([ids[:, 1:], torch.full((batch, 1), -100)], 1)
    return ids, labels


def reference_losses(name: str, steps: int, batch: int, num_mb: int, lr: float = 1e-3, dp: int = 1):
    """Single-process eager run with the engine's loss convention: per-micro-batch mean loss, gradients summed
    over micro-batches and averaged over data-parallel replicas."""
    import torch.nn.functional as F
    model = build_model(name)
    opt = torch.optim.AdamW(model.parameters(), lr=lr)
    out = []
    for step in range(steps):
        ids, labels = make_batch(name, batch, seed=step)
        opt.zero_grad()
        ls = []
        per = ids.shape[0] // dp
        for r in range(dp):
            for ci, cl in zip(ids[r * per:(r + 1) * per].chunk(num_mb), labels[r * per:(r + 1) * per].chunk(num_mb)):
                if name == "mlp":
                    loss = F.mse_loss(model(ci), cl)
                else:
                    logits = model(input_ids=ci, use_cache=False).logits
                    loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), cl.reshape(-1), ignore_index=-100)
                (loss / dp).backward()
                ls.append(loss.item())
        opt.step()
        out.append(sum(ls) / len(ls))
    checksum = float(sum(p.detach().double().abs().sum().item() for p in model.parameters()))
    return out, checksum
