"""Train a model in one given layout for a few steps and print the measured step time (one JSON line from rank 0).

    torchrun --nproc-per-node 8 -m aicomp_b200.fasop.run_layout --model llama3b --tp 1 --dp 4 --pp 2 --mbs 1 --gbs 128

Used by :mod:`aicomp_b200.fasop.validate` to compare the cost model's prediction with reality.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--mbs", type=int, default=1)
    ap.add_argument("--gbs", type=int, default=128)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--tp-backend", default="fused")
    ap.add_argument("--dp-backend", default="fused")
    a = ap.parse_args(argv)
    from transformers import LlamaConfig, LlamaForCausalLM

    from aicomp_b200 import FusedAdamW, Optimus_p, ops
    from .config import MODEL_CONFIGS
    m = MODEL_CONFIGS[a.model]
    S = a.seq_len or m.seq_len
    cfg = LlamaConfig(vocab_size=m.vocab, hidden_size=m.hidden, intermediate_size=m.ffn, num_hidden_layers=m.num_layers,
                      num_attention_heads=m.heads, num_key_value_heads=m.kv_heads, head_dim=m.head_dim, rms_norm_eps=1e-5,
                      max_position_embeddings=max(8192, S), rope_theta=500000.0, tie_word_embeddings=False)
    with torch.device("meta"):
        model = LlamaForCausalLM(cfg)
    per_replica = a.gbs // a.dp
    num_mb = per_replica // a.mbs
    eng = Optimus_p(model, num_mb=num_mb, use_gpu=True, pp_size=a.pp, dp_size=a.dp, tp_size=a.tp, dtype=torch.bfloat16,
                    tp_backend=a.tp_backend, dp_backend=a.dp_backend, cuda_graphs=True)
    opt = FusedAdamW(eng.parameters(), lr=1e-4, grad_scale=1.0 / num_mb, max_grad_norm=1.0,
                     norm_groups={"pp": eng.tpl.pp_group, "tp": eng.tpl.tp_group})
    if eng.dp is not None:
        opt.attach_to_reducer(eng.dp)
    dev = eng.device
    g = torch.Generator().manual_seed(7 + eng.tpl.dp_rank)
    ids = torch.randint(0, m.vocab, (per_replica, S), generator=g).to(dev)
    labels = torch.cat([ids[:, 1:], torch.full((per_replica, 1), -100, device=dev)], 1)

    def step():
        opt.zero_grad()
        eng.run(ids if eng.is_first_stage() else None, labels if eng.is_last_stage() else None, mode="1f1b")
        opt.step()

    for _ in range(a.warmup):
        step()
    if eng.comm.world_size > 1:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.steps):
        step()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / a.steps], device=dev)
    if eng.comm.world_size > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ops.check_errors()
    mem = torch.tensor([torch.cuda.max_memory_allocated() / 2**30], device=dev)
    if eng.comm.world_size > 1:
        dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    if eng.comm.rank == 0:
        print(json.dumps({"layout": {"tp": a.tp, "dp": a.dp, "pp": a.pp, "mbs": a.mbs, "gbs": a.gbs}, "model": a.model, "seq_len": S,
                          "measured_step_s": t.item() / 1e3, "peak_mem_gb": mem.item(),
                          "tokens_per_s": a.gbs * S / (t.item() / 1e3)}), flush=True)
    eng.comm.barrier()


if __name__ == "__main__":
    main()
