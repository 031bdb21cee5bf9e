"""Serving benchmark: Llama-3-8B, continuous batching, paged KV (block 16), Poisson arrivals.

    python bench_serve.py [--requests 1024 --rate 8 --tp 1]            # one replica, colocated
    torchrun --nproc-per-node T bench_serve.py --tp T                  # tensor parallel inside the replica
    torchrun --nproc-per-node 8 bench_serve.py --pd 4                  # 4 prefill GPUs pushing KV pages to 4 decode GPUs

Prompt lengths uniform 128-2048, output lengths uniform 64-512, token ids uniform over the vocabulary, greedy
decoding with EOS disabled, bf16 random-init weights.  Prints one JSON line with decode tokens/s and TTFT.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=1024)
    ap.add_argument("--rate", type=float, default=8.0)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--max-seqs", type=int, default=256)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--fast-clock", action="store_true", help="do not wait for arrivals in real time")
    ap.add_argument("--pd", type=int, default=0, help="prefill/decode disaggregation with this many prefill->decode GPU pairs")
    ap.add_argument("--max-wall", type=float, default=None, help="stop serving after this many seconds")
    a = ap.parse_args()
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM

    from aicomp_b200 import ops
    from aicomp_b200.serve.engine import ServingEngine
    from aicomp_b200.serve.loadgen import make_requests

    cfg = LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=a.layers,
                      num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, max_position_embeddings=8192,
                      rope_theta=500000.0, tie_word_embeddings=False)
    with torch.device("meta"):
        model = LlamaForCausalLM(cfg)
    reqs = make_requests(a.requests, a.rate, seed=0)
    if a.pd:
        import torch.distributed as dist

        from aicomp_b200.serve.pd_engine import run_pd_serving
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        if not dist.is_initialized():
            dist.init_process_group("nccl")
        m = run_pd_serving(model, reqs, a.pd, a.pd, max_seqs=a.max_seqs, max_seq_len=2048 + 512 + 16, max_wall_s=a.max_wall)
        if m is not None:
            print(json.dumps({"metric": "llama3_8b_serving_pd", "decode_tokens_per_s": round(m["decode_tokens_per_s"], 1),
                              "ttft_p50_s": round(m["ttft_p50_s"], 4), "ttft_p99_s": round(m["ttft_p99_s"], 4),
                              "tpot_p50_ms": round(1e3 * m["tpot_p50_s"], 3), "n_gpus": 2 * a.pd, "requests": m["requests"],
                              "wall_s": round(m["wall_s"], 2), "config": {"model": "Llama-3-8B" if a.layers == 32 else f"{a.layers}L",
                              "rate_req_s": a.rate, "prefill_gpus": a.pd, "decode_gpus": a.pd, "kv_block": 16},
                              "dtype": "bf16", "data": "synthetic", "details": m}), flush=True)
        dist.barrier()
        return
    eng = ServingEngine(model, tp_size=a.tp, max_seqs=a.max_seqs, max_seq_len=2048 + 512 + 16, cuda_graphs=not a.no_graphs)
    eng.warmup()
    ops.reset_launch_count()
    m = eng.serve(reqs, realtime=not a.fast_clock, max_wall_s=a.max_wall)
    ops.check_errors()
    if eng.comm.rank == 0:
        print(json.dumps({"metric": "llama3_8b_serving", "decode_tokens_per_s": round(m["decode_tokens_per_s"], 1),
                          "ttft_p50_s": round(m["ttft_p50_s"], 4), "ttft_p99_s": round(m["ttft_p99_s"], 4),
                          "tpot_p50_ms": round(1e3 * m["tpot_p50_s"], 3), "n_gpus": a.tp, "requests": m["requests"],
                          "wall_s": round(m["wall_s"], 2), "config": {"model": "Llama-3-8B" if a.layers == 32 else f"{a.layers}L",
                          "rate_req_s": a.rate, "tp": a.tp, "kv_block": 16, "kv_pages": m["kv_pages"], "cuda_graphs": not a.no_graphs,
                          "peak_running": m["peak_running"]}, "dtype": "bf16", "data": "synthetic", "details": m}), flush=True)


if __name__ == "__main__":
    main()
