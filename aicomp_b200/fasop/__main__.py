"""FASOP command line (flag names follow the reference's fasop/FASOP.py:112-193)."""
from __future__ import annotations

import argparse
import os
import sys
import time

from .config import MODEL_CONFIGS
from .partitioners import PARTITION_METHODS
from .search import FasopConfig, pareto_front, run_strategy_search, save_csv


def parse(argv=None):
    ap = argparse.ArgumentParser(prog="python -m aicomp_b200.fasop", description="Parallelisation strategy search for B200 clusters")
    ap.add_argument("--gpus", nargs="+", required=True, metavar="TYPE N", help="pairs: GPU type and count (nodes, or GPUs if <= one node)")
    ap.add_argument("--model-type", default="llama3b", choices=sorted(MODEL_CONFIGS))
    ap.add_argument("--dataset", default="synthetic")
    ap.add_argument("--gbs", type=int, nargs="+", default=[128])
    ap.add_argument("--gpu-per-node", type=int, default=8)
    ap.add_argument("--precision", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--pp-partition-method", default="minmax", choices=PARTITION_METHODS)
    ap.add_argument("--exhaustive", nargs=4, type=int, metavar=("TP", "DP", "PP", "MBS"), help="evaluate one configuration verbosely")
    ap.add_argument("--pareto", action="store_true")
    ap.add_argument("--make-pareto", action="store_true")
    ap.add_argument("--only-make-pareto", metavar="CSV")
    ap.add_argument("--pareto-title", default="FASOP")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--log-file", default=None)
    ap.add_argument("--add-exp-name", default="")
    ap.add_argument("--no-save-csv", action="store_true")
    ap.add_argument("--profile-dir", default=None)
    ap.add_argument("--top", type=int, default=10)
    ap.add_argument("--placement", default="permutations", choices=["permutations", "cyclic", "grouped"],
                    help="mixed clusters: which orders of the nodes along the pipeline to evaluate")
    return ap.parse_args(argv)


def main(argv=None):
    a = parse(argv)
    if len(a.gpus) % 2:
        raise SystemExit("--gpus takes TYPE N pairs")
    gpus = [(a.gpus[i], int(a.gpus[i + 1])) for i in range(0, len(a.gpus), 2)]
    cfg = FasopConfig(gpus, a.model_type, a.dataset, a.gbs, a.gpu_per_node, a.precision, a.pp_partition_method, a.seq_len,
                      verbose=a.verbose, profile_dir=a.profile_dir, pareto=a.pareto, placement=a.placement)
    if a.exhaustive:
        from .config import ModelConfig
        from .cost import estimate
        from .profiledb import ProfileDB
        tp, dp, pp, mbs = a.exhaustive
        model = MODEL_CONFIGS[a.model_type]
        e = estimate(model, ProfileDB(model, gpus[0][0], a.profile_dir), gpus[0][0], tp, dp, pp, mbs, a.gbs[0], a.pp_partition_method)
        print(f"tp{tp} dp{dp} pp{pp} mbs{mbs}: step {e.step_time:.4f} s, pipe {e.pipe_time:.4f} s, dp {e.dp_cost:.4f} s, "
              f"imbalance {100 * e.imbalance:.2f} %, partition {e.partition}, peak mem {max(e.peak_mem_gb):.1f} GB, oom={e.is_oom}")
        return 0
    exp = f"{a.model_type}_{'_'.join(f'{t}{n}' for t, n in gpus)}{('_' + a.add_exp_name) if a.add_exp_name else ''}_{int(time.time())}"
    jsonl = os.path.join("main_logs", exp + ".jsonl")
    os.makedirs("main_logs", exist_ok=True)
    t0 = time.time()
    results = run_strategy_search(cfg, jsonl)
    dt = time.time() - t0
    print(f"{len(results)} configurations evaluated in {dt:.2f} s")
    print(f"{'rank':>4} {'gbs':>5} {'mbs':>4} {'tp':>3} {'dp':>3} {'pp':>3} {'step(s)':>9} {'samples/s':>10} {'mem(GB)':>8} oom partition")
    for r in results[:a.top]:
        print(f"{r.rank:>4} {r.gbs:>5} {r.mbs:>4} {r.tp:>3} {r.dp:>3} {r.pp:>3} {r.step_time:>9.4f} {r.throughput:>10.2f} "
              f"{r.oom_gpumem:>8.1f} {str(r.is_oom):>5} {r.partition}" + (f" {r.node_type}" if "-" in r.node_type else ""))
    if not a.no_save_csv:
        save_csv(results, os.path.join("main_logs", exp + ".csv"))
    if a.pareto or a.make_pareto:
        from .pareto import save_pareto
        save_pareto(pareto_front(results), os.path.join("main_logs", exp + "_pareto"), a.pareto_title)
    best = next((r for r in results if not r.is_oom), None)
    if best:
        print(f"best: tp{best.tp} dp{best.dp} pp{best.pp} mbs{best.mbs} -> {best.step_time:.4f} s/step")
    return 0


if __name__ == "__main__":
    sys.exit(main())
