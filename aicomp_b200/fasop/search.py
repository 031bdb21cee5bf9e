"""Strategy enumeration and ranking (the role of fasop/FASOP.py:401-889 and fasop/utils.py:119-221)."""
from __future__ import annotations

import csv
import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

from .config import DATASETS, GPU_SPECS, MODEL_CONFIGS, PRICE_PER_NODE_HOUR, ModelConfig
from .cost import Estimate, estimate
from .profiledb import ProfileDB


@dataclass
class FasopConfig:
    gpus: List[Tuple[str, int]]                 # [(type, number of nodes)]
    model_type: str = "llama3b"
    dataset: str = "synthetic"
    gbs: List[int] = field(default_factory=lambda: [128])
    gpu_per_node: int = 8
    precision: int = 16
    pp_partition_method: str = "minmax"
    seq_len: Optional[int] = None
    schedule: str = "1f1b"
    verbose: bool = False
    profile_dir: Optional[str] = None
    pareto: bool = False              # mixed clusters: also evaluate every sub-cluster
    placement: str = "permutations"   # mixed clusters: node orders to try ('permutations', 'cyclic', 'grouped')


@dataclass
class SearchResult:
    gbs: int
    mbs: int
    tp: int
    dp: int
    pp: int
    node_type: str
    gpu_cluster: str
    partition: List[int]
    partition_layers: List[float]
    step_time: float
    throughput: float
    price_per_step: float
    is_oom: bool
    oom_gpumem: float
    iterations: int
    total_time: float
    cost: float
    num_mb: int = 0
    rank: int = 0


def divisors(n: int) -> List[int]:
    return [d for d in range(1, n + 1) if n % d == 0]


def rank2axis(rank: int, pp: int, dp: int, tp: int) -> Tuple[int, int, int]:
    return rank // (dp * tp), (rank // tp) % dp, rank % tp


def axis2rank(stage: int, dp_idx: int, tp_idx: int, dp: int, tp: int) -> int:
    return stage * dp * tp + dp_idx * tp + tp_idx


def enumerate_parallel_strategies(num_gpus: int, gbs: int, num_layers: int, gpus_per_node: int = 8, max_tp: int = 8
                                  ) -> Iterable[Tuple[int, int, int, int]]:
    """(tp, dp, pp, mbs): tp divides the node size, dp divides what is left and the batch, pp <= layers + 2."""
    for tp in [d for d in divisors(num_gpus) if d <= min(max_tp, gpus_per_node)]:
        rest = num_gpus // tp
        for dp in divisors(rest):
            if gbs % dp:
                continue
            pp = rest // dp
            if pp > num_layers + 2:
                continue
            for mbs in divisors(gbs // dp):
                if mbs > 128:
                    continue
                yield tp, dp, pp, mbs


def evaluate(cfg: FasopConfig, model: ModelConfig, gpu: str, num_gpus: int, gbs: int, db: ProfileDB) -> List[SearchResult]:
    out: List[SearchResult] = []
    n_nodes = max(1, num_gpus // cfg.gpu_per_node)
    price_h = PRICE_PER_NODE_HOUR.get(gpu, 0.0) * n_nodes
    iters = max(1, DATASETS.get(cfg.dataset, 131072) // gbs)
    for tp, dp, pp, mbs in enumerate_parallel_strategies(num_gpus, gbs, model.num_layers, cfg.gpu_per_node):
        if model.heads % tp or model.kv_heads % tp or model.ffn % tp:
            continue
        try:
            e: Estimate = estimate(model, db, gpu, tp, dp, pp, mbs, gbs, cfg.pp_partition_method, cfg.gpu_per_node,
                                   cfg.precision // 8, cfg.schedule)
        except ValueError:
            continue
        price_step = price_h / 3600.0 * e.step_time
        out.append(SearchResult(gbs, mbs, tp, dp, pp, gpu, f"{gpu}x{num_gpus}", e.partition, e.partition_layers, e.step_time,
                                gbs / e.step_time, price_step, e.is_oom, max(e.peak_mem_gb), iters, iters * e.step_time,
                                iters * price_step, e.num_mb))
    return out


def evaluate_mixed(cfg: FasopConfig, model: ModelConfig, cluster: List[Tuple[str, int]], gbs: int, dbs: Dict[str, ProfileDB]
                   ) -> List[SearchResult]:
    """A cluster of several node types: every node order (device placement) x every (tp, dp, pp, mbs)."""
    from .device_placement import node_orders, price_per_hour, stage_gpu_types
    out: List[SearchResult] = []
    n_nodes = sum(n for _, n in cluster)
    num_gpus = n_nodes * cfg.gpu_per_node
    iters = max(1, DATASETS.get(cfg.dataset, 131072) // gbs)
    name = "+".join(f"{t}x{n * cfg.gpu_per_node}" for t, n in cluster)
    seen = set()
    for order in node_orders(cluster, cfg.placement):
        price_h = price_per_hour(order, PRICE_PER_NODE_HOUR)
        for tp, dp, pp, mbs in enumerate_parallel_strategies(num_gpus, gbs, model.num_layers, cfg.gpu_per_node):
            if model.heads % tp or model.kv_heads % tp or model.ffn % tp:
                continue
            stages = stage_gpu_types(order, pp, dp, tp, cfg.gpu_per_node)
            key = (tuple(stages), tp, dp, pp, mbs)
            if key in seen:   # different node orders that give every stage the same GPU type are one layout
                continue
            seen.add(key)
            try:
                e = estimate(model, dbs[stages[0]], stages[0], tp, dp, pp, mbs, gbs, cfg.pp_partition_method, cfg.gpu_per_node,
                             cfg.precision // 8, cfg.schedule, stage_gpus=stages, dbs=dbs)
            except ValueError:
                continue
            price_step = price_h / 3600.0 * e.step_time
            out.append(SearchResult(gbs, mbs, tp, dp, pp, "-".join(stages), name, e.partition, e.partition_layers, e.step_time,
                                    gbs / e.step_time, price_step, e.is_oom, max(e.peak_mem_gb), iters, iters * e.step_time,
                                    iters * price_step, e.num_mb))
    return out


def run_strategy_search(cfg: FasopConfig, jsonl_path: Optional[str] = None) -> List[SearchResult]:
    model = MODEL_CONFIGS[cfg.model_type]
    if cfg.seq_len:
        model = ModelConfig(**{**asdict(model), "seq_len": cfg.seq_len})
    results: List[SearchResult] = []
    sink = open(jsonl_path, "w") if jsonl_path else None
    if sink:
        sink.write(json.dumps({"type": "meta", "model": cfg.model_type, "gpus": cfg.gpus, "gbs": cfg.gbs, "time": time.time()}) + "\n")
    if len({g for g, n in cfg.gpus if n > 0}) > 1:
        from .device_placement import cluster_subsets
        for gpu, _ in cfg.gpus:
            if gpu not in GPU_SPECS:
                raise ValueError(f"unknown GPU type {gpu}; known: {sorted(GPU_SPECS)}")
        dbs = {g: ProfileDB(model, g, cfg.profile_dir) for g, _ in cfg.gpus}
        for sub in cluster_subsets(cfg.gpus, cfg.pareto):
            for gbs in cfg.gbs:
                if len(sub) == 1:
                    g, n = sub[0]
                    rs = evaluate(cfg, model, g, n * cfg.gpu_per_node, gbs, dbs[g])
                else:
                    rs = evaluate_mixed(cfg, model, sub, gbs, dbs)
                results.extend(rs)
                if sink:
                    for r in rs:
                        sink.write(json.dumps(asdict(r)) + "\n")
        if sink:
            sink.close()
        results.sort(key=lambda r: (r.is_oom, r.total_time))
        for i, r in enumerate(results):
            r.rank = i + 1
        return results
    for gpu, nodes in cfg.gpus:
        if gpu not in GPU_SPECS:
            raise ValueError(f"unknown GPU type {gpu}; known: {sorted(GPU_SPECS)}")
        num_gpus = nodes if nodes <= cfg.gpu_per_node and len(cfg.gpus) == 1 and nodes in (1, 2, 4, 8) else nodes * cfg.gpu_per_node
        db = ProfileDB(model, gpu, cfg.profile_dir)
        for gbs in cfg.gbs:
            rs = evaluate(cfg, model, gpu, num_gpus, gbs, db)
            results.extend(rs)
            if sink:
                for r in rs:
                    sink.write(json.dumps(asdict(r)) + "\n")
    if sink:
        sink.close()
    results.sort(key=lambda r: (r.is_oom, r.total_time))
    for i, r in enumerate(results):
        r.rank = i + 1
    return results


CSV_COLUMNS = ["index", "gbs", "mbs", "tp", "dp", "pp", "node_type", "gpu_cluster", "partition", "partition_layers", "step_time(s)",
               "throughput(samples/s)", "price_per_step($)", "is_oom", "oom_gpumem(GB)", "iterations", "total_time(s)",
               "total_time(h)", "cost($)", "rank"]


def save_csv(results: List[SearchResult], path: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(CSV_COLUMNS)
        for i, r in enumerate(results):
            w.writerow([i, r.gbs, r.mbs, r.tp, r.dp, r.pp, r.node_type, r.gpu_cluster, r.partition, r.partition_layers,
                        f"{r.step_time:.6f}", f"{r.throughput:.4f}", f"{r.price_per_step:.6f}", r.is_oom, f"{r.oom_gpumem:.2f}",
                        r.iterations, f"{r.total_time:.2f}", f"{r.total_time / 3600:.4f}", f"{r.cost:.2f}", r.rank])


def pareto_front(results: List[SearchResult]) -> List[SearchResult]:
    """Skyline over (total time, cost) among non-OOM results."""
    pts = sorted([r for r in results if not r.is_oom], key=lambda r: (r.total_time, r.cost))
    front, best_cost = [], float("inf")
    for r in pts:
        if r.cost < best_cost:
            front.append(r)
            best_cost = r.cost
    return front
