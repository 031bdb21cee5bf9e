"""Continuous-batching server loop on synthetic traffic (paged KV cache, Poisson arrivals); prints TTFT and throughput."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aicomp_b200.serve.engine import ServingEngine  # noqa: E402
from aicomp_b200.serve.loadgen import make_requests  # noqa: E402


def main():
    from transformers import LlamaConfig, LlamaForCausalLM
    cpu = "--cpu" in sys.argv
    cfg = LlamaConfig(num_hidden_layers=4, hidden_size=1024, num_attention_heads=8, num_key_value_heads=2, intermediate_size=2816,
                      vocab_size=32000, max_position_embeddings=4096, tie_word_embeddings=False)
    torch.manual_seed(0)
    eng = ServingEngine(LlamaForCausalLM(cfg), use_gpu=not cpu, max_seqs=64, max_seq_len=1024, num_pages=512 if cpu else None)
    reqs = make_requests(32, rate_per_s=16.0, prompt_range=(16, 256), output_range=(8, 64), vocab=cfg.vocab_size)
    eng.warmup(max_batch=32) if not cpu else None
    m = eng.serve(reqs, realtime=not cpu)
    print({k: (round(v, 4) if isinstance(v, float) else v) for k, v in m.items()})


if __name__ == "__main__":
    main()
