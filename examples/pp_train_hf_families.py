"""Pipeline-parallel training of the other HuggingFace families the reference ships examples for, on synthetic data.

    torchrun --nproc-per-node 2 examples/pp_train_hf_families.py --model vit [--cpu]

``--model``: gpt-neo, gptj, bert, electra, opt, vit, whisper, gpt2-seq-cls, qwen-moe, synthetic (a plain ``nn.Module``
of ten linear layers with an MSE loss).  One script instead of the reference's one file per model
(opt_prime/examples/pp_train_{gpt-neo,gptj,bert,electra,opt,vit,whisper,gpt2_seq-cls,qwen_moe,synthetic}.py); the
sizes are small so that every model also runs on CPU/gloo, pass ``--hidden/--layers`` for larger ones.
"""
import argparse
import os
import sys
import time

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from opt_prime.opti_pri import Optimus_p  # noqa: E402


def build(name: str, hidden: int, layers: int, heads: int, vocab: int):
    """Returns (model, make_batch(generator) -> (data, labels), extra engine kwargs)."""
    import transformers as T
    ffn = 4 * hidden

    def tokens(g, b=8, s=64):
        return torch.randint(1, vocab, (b, s), generator=g)
    if name == "synthetic":
        model = nn.Sequential(*[m for _ in range(10) for m in (nn.Linear(hidden, hidden), nn.ReLU())])
        return model, lambda g: (torch.randn(8, hidden, generator=g), torch.randn(8, hidden, generator=g)), {}
    if name == "vit":
        cfg = T.ViTConfig(hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads, intermediate_size=ffn, image_size=64,
                          patch_size=8, num_labels=10)
        return (T.ViTForImageClassification(cfg),
                lambda g: (torch.randn(8, 3, 64, 64, generator=g), torch.randint(0, 10, (8,), generator=g)), {})
    if name == "whisper":
        cfg = T.WhisperConfig(vocab_size=vocab, d_model=hidden, encoder_layers=layers // 2, decoder_layers=layers // 2,
                              encoder_attention_heads=heads, decoder_attention_heads=heads, encoder_ffn_dim=ffn, decoder_ffn_dim=ffn,
                              num_mel_bins=16, max_source_positions=32, max_target_positions=64, pad_token_id=0, bos_token_id=1,
                              eos_token_id=2, decoder_start_token_id=1)

        def batch(g):
            dec = tokens(g, 8, 33)
            return {"input_features": torch.randn(8, 16, 64, generator=g), "decoder_input_ids": dec[:, :-1]}, dec[:, 1:]
        return T.WhisperForConditionalGeneration(cfg), batch, {"input_names": ["input_features", "decoder_input_ids"]}
    if name == "gpt2-seq-cls":
        cfg = T.GPT2Config(vocab_size=vocab, n_embd=hidden, n_layer=layers, n_head=heads, n_positions=128, num_labels=4, pad_token_id=0)
        return T.GPT2ForSequenceClassification(cfg), lambda g: (tokens(g), torch.randint(0, 4, (8,), generator=g)), {}
    causal = {
        "gpt-neo": lambda: T.GPTNeoForCausalLM(T.GPTNeoConfig(vocab_size=vocab, hidden_size=hidden, num_layers=layers, num_heads=heads,
                                                              attention_types=[[["global", "local"], layers // 2]],
                                                              max_position_embeddings=128, window_size=32)),
        "gptj": lambda: T.GPTJForCausalLM(T.GPTJConfig(vocab_size=vocab, n_embd=hidden, n_layer=layers, n_head=heads,
                                                       rotary_dim=hidden // heads // 2, n_positions=128)),
        "opt": lambda: T.OPTForCausalLM(T.OPTConfig(vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
                                                    num_attention_heads=heads, ffn_dim=ffn, max_position_embeddings=128,
                                                    word_embed_proj_dim=hidden)),
        "qwen-moe": lambda: T.Qwen2MoeForCausalLM(T.Qwen2MoeConfig(
            vocab_size=vocab, hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers, num_attention_heads=heads,
            num_key_value_heads=max(1, heads // 2), moe_intermediate_size=hidden, shared_expert_intermediate_size=2 * hidden,
            num_experts=4, num_experts_per_tok=2, max_position_embeddings=128)),
    }
    masked = {
        "bert": lambda: T.BertForMaskedLM(T.BertConfig(vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
                                                       num_attention_heads=heads, intermediate_size=ffn, max_position_embeddings=128)),
        "electra": lambda: T.ElectraForMaskedLM(T.ElectraConfig(vocab_size=vocab, embedding_size=hidden // 2, hidden_size=hidden,
                                                                num_hidden_layers=layers, num_attention_heads=heads,
                                                                intermediate_size=ffn, max_position_embeddings=128)),
    }
    if name in causal:
        def batch(g):
            t = tokens(g, 8, 65)
            return t[:, :-1], t[:, 1:]
        return causal[name](), batch, {}
    if name in masked:
        def batch(g):  # masked-LM: predict 15 % of the positions, ignore the rest
            t = tokens(g)
            labels = t.clone()
            labels[torch.rand(t.shape, generator=g) > 0.15] = -100
            return t, labels
        return masked[name](), batch, {}
    raise SystemExit(f"unknown model {name}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="opt")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--mode", default="1f1b", choices=["gpipe", "1f1b"])
    ap.add_argument("--hidden", type=int, default=128)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--vocab", type=int, default=1024)
    ap.add_argument("--dynamo-capture", action="store_true")
    a = ap.parse_args()
    torch.manual_seed(0)
    model, make_batch, extra = build(a.model, a.hidden, a.layers, a.heads, a.vocab)
    partitioner = "hierarchical" if a.model == "qwen-moe" else "auto"   # MoE graphs: group modules by block first
    engine = Optimus_p(model, num_mb=4, use_gpu=not a.cpu, dynamo_capture=a.dynamo_capture, partitioner=partitioner, **extra)
    engine.train()
    optimizer = torch.optim.AdamW(engine.parameters(), lr=3e-4)
    engine.optimizer = optimizer
    g = torch.Generator().manual_seed(0)
    for step in range(a.steps):
        data, labels = make_batch(g)
        t0 = time.time()
        labels = engine.move_labels2last_stage(labels)
        optimizer.zero_grad()
        engine.run(data if engine.is_first_stage() else None, labels, mode=a.mode)
        loss = engine.get_loss()
        torch.nn.utils.clip_grad_norm_(engine.parameters(), 1.0)
        optimizer.step()
        if engine.is_last_stage():
            print(f"{a.model} step {step}: loss {sum(loss) / len(loss):.4f}  {1e3 * (time.time() - t0):.0f} ms/batch", flush=True)
    engine.comm.barrier()


if __name__ == "__main__":
    main()
