"""Headline benchmark: Llama-3-8B training throughput (tokens/s per box) through the public engine API.

Config (weak scaling, 8 sequences of 2048 tokens per GPU per step, micro-batch 1):
  N=1  pp1 dp1  global batch  8      N=4  pp2 dp2  global batch 32
  N=2  pp2 dp1  global batch 16      N=8  pp2 dp4  global batch 64  (the named PP=2 x DP=4, 1F1B, gbs 64 config)
bf16 weights + fp32 master / AdamW, synthetic uniform tokens, random init.  Every step copies that step's
token ids and labels from pinned host memory, runs forward/backward/optimizer through ``Optimus_p.run`` and
``FusedAdamW.step`` and reads the loss back to the host.  ``--impl reference`` runs the same metric through the
reference's own code if it is installed under ``baseline/_ref``.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOKENS_PER_S = None  # the reference publishes no throughput number


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "library"],
                    help="'library': the same engine with its kernels off - eager HF modules on cuBLAS / cuDNN SDPA / NCCL with "
                         "fp32 parameters under bf16 autocast and torch.optim.AdamW, i.e. what the reference's stock path does")
    ap.add_argument("--layers", type=int, default=32, help="debug only: fewer layers make the result INVALID as a bench value")
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--seqs-per-gpu", type=int, default=8)
    ap.add_argument("--dp-backend", default="fused")
    ap.add_argument("--attn", default="kernel", choices=["kernel", "sdpa"],
                    help="'sdpa': library attention (cuDNN) instead of the flash kernels of this framework, for an A/B comparison")
    ap.add_argument("--no-graphs", action="store_true", help="issue every kernel from Python instead of replaying CUDA graphs")
    ap.add_argument("--layout", default="", help="pp,dp,tp override, e.g. 2,1,4 with --seq 4096 --seqs-per-gpu 4 for the "
                                                 "TP4 x PP2 config (the metric line then names that parallelism)")
    ap.add_argument("--tp-backend", default="fused")
    return ap.parse_args()


def layout_for(n):
    return {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (2, 4)}[n]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._t = None

    def _run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                parts = [p.strip() for p in out.split(",")]
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
                for n, v in zip(names, parts[2:]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.2)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def run_ours(a):
    import torch
    import torch.distributed as dist
    from transformers import LlamaConfig, LlamaForCausalLM

    from aicomp_b200 import FusedAdamW, Optimus_p, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {a.gpus}")
    pp, dp = layout_for(a.gpus)
    tp = 1
    if a.layout:
        pp, dp, tp = (int(v) for v in a.layout.split(","))
        if pp * dp * tp != a.gpus:
            raise SystemExit(f"--layout {a.layout} does not use {a.gpus} GPUs")
    cfg = LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=a.layers,
                      num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, max_position_embeddings=8192,
                      rope_theta=500000.0, tie_word_embeddings=False, attention_bias=False)
    with torch.device("meta"):
        model = LlamaForCausalLM(cfg)
    seqs_per_replica = a.seqs_per_gpu * a.gpus // dp
    num_mb = seqs_per_replica  # micro-batch 1
    library = a.impl == "library"
    if a.attn == "sdpa":
        from aicomp_b200.ops import flash
        flash.TRAINING_USES_KERNEL = False
    if library:
        eng = Optimus_p(model, num_mb=num_mb, use_gpu=True, pp_size=pp, dp_size=dp, tp_size=tp, dtype=torch.float32,
                        fused_kernels=False, dp_backend="nccl", tp_backend="nccl", pp_backend="nccl", cuda_graphs=False)
        opt = torch.optim.AdamW(eng.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    else:
        eng = Optimus_p(model, num_mb=num_mb, use_gpu=True, pp_size=pp, dp_size=dp, tp_size=tp, dtype=torch.bfloat16,
                        dp_backend=a.dp_backend, tp_backend=a.tp_backend, cuda_graphs=not a.no_graphs)
        opt = FusedAdamW(eng.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, grad_scale=1.0 / num_mb, max_grad_norm=1.0,
                         norm_groups={"pp": eng.tpl.pp_group, "tp": eng.tpl.tp_group if tp > 1 else None})
    dev = eng.device
    eng.optimizer = opt
    if eng.dp is not None and not library:
        opt.attach_to_reducer(eng.dp)
    S = a.seq
    gbs = a.seqs_per_gpu * a.gpus
    g = torch.Generator().manual_seed(1234 + eng.tpl.dp_rank)
    n_batches = a.warmup + a.steps  # a fresh synthetic batch every step
    host_ids = [torch.randint(0, cfg.vocab_size, (seqs_per_replica, S), generator=g).pin_memory() for _ in range(n_batches)]
    host_labels = [torch.cat([t[:, 1:], torch.full((seqs_per_replica, 1), -100, dtype=torch.long)], 1).pin_memory() for t in host_ids]
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    first, last = eng.is_first_stage(), eng.is_last_stage()

    def step(i):
        ids = host_ids[i % n_batches].to(dev, non_blocking=True) if first else None
        labels = host_labels[i % n_batches].to(dev, non_blocking=True) if last else None  # labels go straight to the last stage
        opt.zero_grad()
        if library:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                eng.run(ids, labels, mode="1f1b")
            eng.clip_grad_norm_(1.0)
        else:
            eng.run(ids, labels, mode="1f1b")
        opt.step()
        if last:
            loss_host.copy_(eng.get_loss_tensor().reshape(1), non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(a.warmup):
        step(i)
    barrier()
    ops.check_errors()
    ops.reset_launch_count()
    sampler = ClockSampler(eng.comm.local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.perf_counter()
    ev0.record()
    for i in range(a.steps):
        step(a.warmup + i)
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1)
    t = torch.tensor([ms, wall * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    launches = torch.tensor([float(ops.launch_count())], device=dev)
    if world > 1:
        dist.all_reduce(launches)
    ops.check_errors()
    ms_dev, ms_wall = t[0].item(), t[1].item()
    tokens = gbs * S * a.steps
    if world > 1:
        # loss lives on the last stage; bring one copy to rank 0 for the report
        lt = torch.tensor([loss_host.item() if last else 0.0], device=dev)
        dist.all_reduce(lt, op=dist.ReduceOp.MAX)
        loss_val = lt.item()
    else:
        loss_val = loss_host.item()
    if eng.comm.rank == 0:
        ms_step = ms_dev / a.steps
        value = tokens / (ms_dev / 1e3)
        e2e = tokens / (ms_wall / 1e3)
        res = {
            "metric": "llama3_8b_train_tokens_per_s_per_box", "value": round(value, 1), "unit": "tokens/s", "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms_step, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
            "impl": "library stand-in (this engine, kernels off)" if library else "ours",
            "config": {"model": "Llama-3-8B" if a.layers == 32 else f"Llama-3-8B-width/{a.layers}L (INVALID: reduced)",
                       "global_batch": gbs, "seq_len": S, "micro_batch": 1, "num_microbatches": num_mb,
                       "parallelism": f"pp{pp}xdp{dp}" + (f"xtp{tp}" if tp > 1 else ""), "schedule": "1f1b", "optimizer": "torch AdamW on fp32 parameters, bf16 autocast" if library else "AdamW fp32 master + bf16 weights",
                       "l2": "inputs larger than L2: every step streams >100 GB of weights, gradients and optimizer state"},
            "clocks": clocks,
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(2 * gbs * S * 8), "d2h_bytes_per_step": 4,
                    "timing": "host wall clock around the same steps incl. pinned H2D of ids+labels and D2H of the loss"},
            "gpu_launches": int(launches.item()),
            "final_loss": round(loss_val, 4),
        }
        print(json.dumps(res), flush=True)
    barrier()
    if world > 1:
        dist.destroy_process_group()


def run_reference(a):
    from baseline.reference_arm import run_reference_arm
    run_reference_arm(a)


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
