"""Reference arm of the benchmark: the UNMODIFIED reference engine on the same metric and config.

``baseline/_ref/opt_prime`` is a verbatim copy of the reference's ``opt_prime/opt_prime`` package (the reference has
no ``setup.py`` / ``pyproject.toml``, so ``pip install --target baseline/_ref`` cannot produce it; the copy is made by
``python baseline/reference_arm.py --install``).  The reference imports ``transformers.utils.fx`` at module level,
which current ``transformers`` no longer ships; a stand-in module with the two names it imports is registered in
``sys.modules`` before the import (nothing in the reference is edited) and the engine is driven through its own
``torch.export`` capture path (``dynamo_capture=True``), its own 1F1B scheduler, torch DDP and NCCL, with
``torch.autocast(bf16)`` and a user-side ``torch.optim.AdamW`` exactly as its demo script does
(opt_prime/demo/pp_train_llama-8b.py:154-155).  When that cannot run, one JSON line says why and the exit code is 0.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def install() -> str:
    src = os.path.join(os.environ.get("AICOMP_REFERENCE_TREE", ""), "opt_prime", "opt_prime")
    dst = os.path.join(REF, "opt_prime")
    if not os.path.isdir(src):
        return "reference tree not mounted (set AICOMP_REFERENCE_TREE to its root)"
    os.makedirs(REF, exist_ok=True)
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst)
    return "ok"


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _shim_transformers_fx() -> None:
    """``transformers.utils.fx`` is imported by the reference for its HFTracer path only; the export path never uses it."""
    if "transformers.utils.fx" in sys.modules:
        return
    import transformers.utils
    m = types.ModuleType("transformers.utils.fx")

    class HFTracer:  # noqa: D401 - placeholder: the symbolic-trace path of the reference is not available here
        def __init__(self, *a, **k):
            raise RuntimeError("transformers.utils.fx.HFTracer is not available in this transformers release")
    m.HFTracer = HFTracer
    m._SUPPORTED_MODELS = ()
    sys.modules["transformers.utils.fx"] = m
    transformers.utils.fx = m


def run_reference_arm(a) -> None:
    if not os.path.isdir(os.path.join(REF, "opt_prime")):
        return _unavailable("reference is not pip-installable (no setup.py/pyproject.toml) and baseline/_ref/opt_prime is absent")
    import torch
    if not torch.cuda.is_available():
        return _unavailable("the reference engine exits when no GPU is present (opt_prime/opt_prime/opti_pri.py:382-388)")
    try:
        _shim_transformers_fx()
        sys.path.insert(0, REF)
        from opt_prime.opti_pri import Optimus_p  # the reference's own class
    except BaseException as e:  # the reference calls sys.exit() on some failures
        return _unavailable(f"reference import failed: {type(e).__name__}: {str(e)[:200]}")
    try:
        _run(a, torch, Optimus_p)
    except BaseException as e:
        import traceback
        tb = traceback.format_exc().strip().splitlines()[-1][:240]
        _unavailable(f"reference run failed: {type(e).__name__}: {tb}")


def _run(a, torch, Optimus_p) -> None:
    import torch.distributed as dist
    from transformers import LlamaConfig, LlamaForCausalLM
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pp, dp = {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (2, 4)}[a.gpus]
    cfg = LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=a.layers,
                      num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, max_position_embeddings=8192,
                      rope_theta=500000.0, tie_word_embeddings=False, attention_bias=False)
    torch.manual_seed(0)
    cfg._attn_implementation = "sdpa"
    model = LlamaForCausalLM(cfg)          # fp32 on the host, as the reference's examples build it
    seqs_per_replica = a.seqs_per_gpu * a.gpus // dp
    num_mb = seqs_per_replica
    eng = Optimus_p(model, num_mb, use_gpu=True, pp_size=pp, dp_size=dp, tp_size=1, dynamo_capture=True, activation_ckpt=False)
    eng.train()
    eng.optimizer = torch.optim.AdamW(eng.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
    S, gbs = a.seq, a.seqs_per_gpu * a.gpus
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    g = torch.Generator().manual_seed(1234)
    n_batches = a.warmup + a.steps
    ids_host = [torch.randint(0, cfg.vocab_size, (seqs_per_replica, S), generator=g).pin_memory() for _ in range(n_batches)]

    def step(i):
        data = labels = None
        if eng.is_first_stage():
            data = ids_host[i]
            labels = torch.cat([data[:, 1:], torch.full((seqs_per_replica, 1), -100, dtype=torch.long)], 1)
        labels = eng.move_labels2last_stage(labels)
        eng.optimizer.zero_grad()
        with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
            eng.run(data, labels, mode="1f1b")
        loss = eng.get_loss() if eng.is_last_stage() else None
        torch.nn.utils.clip_grad_norm_(eng.parameters(), 1.0)
        eng.optimizer.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for i in range(a.warmup):
        step(i)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    loss = None
    for i in range(a.steps):
        loss = step(a.warmup + i)
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    t = torch.tensor([ev0.elapsed_time(ev1), wall * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if int(os.environ.get("RANK", "0")) == 0:
        tokens = gbs * S * a.steps
        print(json.dumps({
            "metric": "llama3_8b_train_tokens_per_s_per_box", "value": round(tokens / (t[0].item() / 1e3), 1), "unit": "tokens/s",
            "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(t[0].item() / a.steps, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 autocast over fp32 weights",
            "data": "synthetic uniform token ids, random-init weights", "impl": "reference",
            "config": {"model": "Llama-3-8B" if a.layers == 32 else f"{a.layers}L (INVALID: reduced)", "global_batch": gbs, "seq_len": S,
                       "parallelism": f"pp{pp}xdp{dp}", "schedule": "1f1b", "capture": "torch.export (dynamo_capture=True)"},
            "e2e": {"value": round(tokens / (t[1].item() / 1e3), 1), "unit": "tokens/s"}}), flush=True)


if __name__ == "__main__":
    if "--install" in sys.argv:
        print(install())
