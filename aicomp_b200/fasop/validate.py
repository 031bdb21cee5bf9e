"""Predicted vs measured: search, then run the top-k predicted layouts on the local GPUs and compare step times.

    python -m aicomp_b200.fasop.validate --model llama3b --gbs 128 --gpus 8 --top 3

Each layout is launched with ``torch.distributed.run`` (one process per GPU, rendezvous on 127.0.0.1) through
:mod:`aicomp_b200.fasop.run_layout`.  Prints a table and writes ``fasop_validation.json``.  The reference never
checks its cost model against measurements in-repo.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys

from .search import FasopConfig, run_strategy_search


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3b")
    ap.add_argument("--gbs", type=int, default=128)
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--gpu-type", default="B200")
    ap.add_argument("--top", type=int, default=3)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--method", default="minmax")
    ap.add_argument("--port", type=int, default=29731)
    ap.add_argument("--out", default="fasop_validation.json")
    ap.add_argument("--distinct", action="store_true", help="skip layouts that differ only in micro-batch size")
    a = ap.parse_args(argv)
    res = [r for r in run_strategy_search(FasopConfig([(a.gpu_type, a.gpus)], a.model, gbs=[a.gbs], pp_partition_method=a.method))
           if not r.is_oom]
    picked, seen = [], set()
    for r in res:
        key = (r.tp, r.dp, r.pp)
        if a.distinct and key in seen:
            continue
        seen.add(key)
        picked.append(r)
        if len(picked) == a.top:
            break
    rows = []
    for i, r in enumerate(picked):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", str(a.port + i), "-m", "aicomp_b200.fasop.run_layout", "--model", a.model, "--tp", str(r.tp), "--dp",
               str(r.dp), "--pp", str(r.pp), "--mbs", str(r.mbs), "--gbs", str(r.gbs), "--steps", str(a.steps)]
        p = subprocess.run(cmd, capture_output=True, text=True, timeout=1200)
        line = next((l for l in reversed(p.stdout.splitlines()) if l.startswith("{")), None)
        if p.returncode != 0 or line is None:
            rows.append({"layout": {"tp": r.tp, "dp": r.dp, "pp": r.pp, "mbs": r.mbs}, "predicted_step_s": r.step_time,
                         "error": (p.stderr or p.stdout)[-600:]})
            continue
        m = json.loads(line)
        m["predicted_step_s"] = r.step_time
        m["predicted_rank"] = r.rank
        m["ratio_measured_over_predicted"] = m["measured_step_s"] / r.step_time
        rows.append(m)
    print(f"{'rank':>4} {'tp':>3} {'dp':>3} {'pp':>3} {'mbs':>4} {'predicted(s)':>13} {'measured(s)':>12} {'ratio':>6}")
    for m in rows:
        l = m["layout"]
        if "error" in m:
            print(f"{'-':>4} {l['tp']:>3} {l['dp']:>3} {l['pp']:>3} {l['mbs']:>4} {m['predicted_step_s']:>13.4f}   FAILED")
        else:
            print(f"{m['predicted_rank']:>4} {l['tp']:>3} {l['dp']:>3} {l['pp']:>3} {l['mbs']:>4} {m['predicted_step_s']:>13.4f} "
                  f"{m['measured_step_s']:>12.4f} {m['ratio_measured_over_predicted']:>6.2f}")
    with open(a.out, "w") as f:
        json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
