"""Explicit prefill / decode loop on a pipeline (and tensor) parallel Llama, with timing of the two phases.

    torchrun --nproc-per-node 2 examples/pp_generation_llama.py --pp-size 2 [--cpu]

The loop that ``Optimus_Inference.generate`` hides, written out with ``ScheduleGeneration.prefill`` and ``decode_step``
as the reference's examples/pp_generation_llama.py:247-443 does: one prefill over the prompt fills the KV cache, then one
token per step; the sampled token travels from the last stage back to the first.
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from opt_prime.inference import Optimus_Inference  # noqa: E402
from opt_prime.schedule_infer import ScheduleGeneration  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--pp-size", type=int, default=1)
    ap.add_argument("--tp-size", type=int, default=1)
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=48)
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    from transformers import LlamaConfig, LlamaForCausalLM
    from aicomp_b200.inference import sample_token
    cfg = LlamaConfig(num_hidden_layers=8, hidden_size=1024, num_attention_heads=8, num_key_value_heads=4, intermediate_size=2816,
                      vocab_size=32000, max_position_embeddings=2048, tie_word_embeddings=False)
    torch.manual_seed(0)
    eng = Optimus_Inference(LlamaForCausalLM(cfg), use_gpu=not a.cpu, pp_size=a.pp_size, tp_size=a.tp_size, use_kv_cache=True,
                            dtype=torch.float32 if a.cpu else torch.bfloat16)
    gen = ScheduleGeneration(eng)
    first, last = eng.is_first_stage(), eng.is_last_stage()
    B, S0 = 2, a.prompt_len
    prompt = torch.randint(0, cfg.vocab_size, (B, S0), generator=torch.Generator().manual_seed(1)).to(eng.device)
    eng._ensure_cache(B)
    eng.clear_kv_cache()

    def sync():
        if not a.cpu:
            torch.cuda.synchronize()

    sync(); t0 = time.perf_counter()
    logits = gen.prefill(prompt if first else None)
    token = sample_token(logits, 1.0, 0, 1.0, False) if last else None
    token, _ = eng._next_token_exchange(token, False, B)
    sync(); t_prefill = time.perf_counter() - t0
    out = [token]
    t0 = time.perf_counter()
    for step in range(1, a.max_new_tokens):
        logits = gen.decode_step(token if first else None, S0 + step - 1)
        token = sample_token(logits, 1.0, 0, 1.0, False) if last else None
        token, _ = eng._next_token_exchange(token, False, B)
        out.append(token)
    sync(); t_decode = time.perf_counter() - t0
    if eng.is_output_rank():
        ids = torch.stack(out, 1)
        print(f"prefill {S0} tokens x {B}: {1e3 * t_prefill:.1f} ms;  decode {a.max_new_tokens - 1} steps: "
              f"{1e3 * t_decode / max(1, a.max_new_tokens - 1):.2f} ms/step, {B * (a.max_new_tokens - 1) / t_decode:.1f} tokens/s")
        print("first sequence:", ids[0].tolist()[:16], "...")
    eng.free_kv_cache()
    eng.barrier()


if __name__ == "__main__":
    main()
