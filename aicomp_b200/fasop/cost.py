"""Cost model: node compute costs from the profile database, communication from an alpha-beta model, memory.

Structure of the reference's ``FASOP.predict`` (fasop/estimate.py:645-890): per-node execution cost, per-cut
transfer cost, partition, 1F1B simulation, data-parallel all-reduce, embedding synchronisation, peak memory
against the device limit.  Differences: backward costs are measured (not 2x forward), the data-parallel cost uses
each stage's own parameter count (the reference uses stage 0's for all, estimate.py:578-592), bandwidths are
NVSwitch-uniform alpha-beta terms, tensor-parallel collectives are counted per layer, and the optimizer step is
included.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

from .config import GPU_SPECS, NODE_TYPES, ModelConfig
from .partitioners import partition, partition_hetero, stage_costs
from .profiledb import ProfileDB
from .sim1f1b import simulate

BYTES_PARAM_STATE = 18  # bf16 weight (2) + fp32 master, m, v (12) + fp32 main gradient (4)


@dataclass
class Estimate:
    step_time: float
    stage_fwd: List[float]
    stage_bwd: List[float]
    partition: List[int]
    partition_layers: List[float]
    pipe_time: float
    dp_cost: float
    tp_cost_per_mb: float
    opt_cost: float
    peak_mem_gb: List[float]
    is_oom: bool
    num_mb: int
    imbalance: float
    details: Dict[str, float] = field(default_factory=dict)


def p2p_time(nbytes: float, spec: Dict[str, float], inter_node: bool = False) -> float:
    bw = spec["inter_node"] if inter_node else spec["intra_p2p"]
    return spec["latency"] + nbytes / bw


def allreduce_time(nbytes: float, n: int, spec: Dict[str, float], inter_node: bool = False, fused: bool = True) -> float:
    if n <= 1:
        return 0.0
    bus = spec.get("fused_allreduce_bus" if fused else "intra_allreduce_bus", spec["intra_allreduce_bus"])
    if inter_node:
        bus = spec["inter_node"]
    return 3 * spec["latency"] + 2.0 * (n - 1) / n * nbytes / bus


def estimate(model: ModelConfig, db: ProfileDB, gpu: str, tp: int, dp: int, pp: int, mbs: int, gbs: int,
             method: str = "minmax", gpus_per_node: int = 8, precision_bytes: int = 2, schedule: str = "1f1b",
             sequence_parallel: bool = True, stage_gpus: Optional[List[str]] = None,
             dbs: Optional[Dict[str, ProfileDB]] = None) -> Estimate:
    """``stage_gpus`` (one GPU type per pipeline stage, with ``dbs`` holding a profile database per type) switches to
    the heterogeneous model: every stage pays its own GPU's node costs, memory limit, all-reduce and optimizer
    bandwidth, and a transfer between two stages runs at the slower side's link speed."""
    if stage_gpus is not None and len(set(stage_gpus)) > 1:
        return _estimate_hetero(model, dbs or {}, stage_gpus, tp, dp, pp, mbs, gbs, gpus_per_node, precision_bytes, schedule,
                                sequence_parallel)
    if stage_gpus:
        gpu = stage_gpus[0]
        db = (dbs or {}).get(gpu, db)
    spec = GPU_SPECS[gpu]
    if gbs % (dp * mbs):
        raise ValueError("gbs must be divisible by dp * mbs")
    num_mb = gbs // (dp * mbs)
    seq = model.node_sequence()
    f_node, b_node = db.node_times(tp, mbs)
    col = {n: i for i, n in enumerate(NODE_TYPES)}
    f_cost = np.array([f_node[col[n]] for n in seq])
    b_cost = np.array([b_node[col[n]] for n in seq])
    tokens = mbs * model.seq_len
    # tensor-parallel collectives per layer and micro-batch: AG + RS around attention and around the MLP, each way
    tp_bytes = tokens * model.hidden * precision_bytes
    tp_layer = 0.0
    if tp > 1:
        per_coll = spec["latency"] + (tp - 1) / tp * tp_bytes / spec["intra_p2p"]
        tp_layer = 4 * per_coll * 0.35  # fused AG->GEMM / GEMM->RS kernels hide most of the transfer behind the math
        for i, n in enumerate(seq):
            if n in ("attn_o", "mlp_down"):
                f_cost[i] += tp_layer / 2
                b_cost[i] += tp_layer / 2
    total = f_cost + b_cost
    # transfer across a cut placed after node i
    world = tp * dp * pp
    inter = world > gpus_per_node and pp > 1 and (tp * dp) >= gpus_per_node
    cut_bytes = np.array([tokens * model.cut_elems(n, tp, sequence_parallel) * precision_bytes for n in seq])
    comm = np.array([p2p_time(b, spec, inter) for b in cut_bytes])
    sizes = partition(method, total, pp, layer_level=(tp > 1), num_mb=num_mb, comm=comm)
    sf, sb = stage_costs(f_cost, sizes), stage_costs(b_cost, sizes)
    bounds = np.cumsum(sizes)[:-1]
    send = [float(comm[c - 1]) for c in bounds]
    ends, _ = simulate(sf, sb, send, send, num_mb, schedule)
    pipe_time = max(ends)
    # per-stage parameters -> data-parallel all-reduce of fp32 gradients, optimizer step, memory
    stage_params, stage_act = [], []
    i = 0
    for n_nodes in sizes:
        nodes = seq[i:i + n_nodes]
        stage_params.append(sum(model.node_params_sharded(n, tp) for n in nodes))
        stage_act.append(sum(model.node_act_elems(n, tp) for n in nodes) * tokens * precision_bytes)
        i += n_nodes
    dp_inter = dp * tp > gpus_per_node
    dp_costs = [allreduce_time(p * 4, dp, spec, dp_inter) for p in stage_params]
    opt_costs = [p * 30.0 / (0.8 * spec["hbm"]) for p in stage_params]
    stage_total = [e + d + o for e, d, o in zip(ends, dp_costs, opt_costs)]
    step = max(stage_total)
    mem = []
    for s, (p, a) in enumerate(zip(stage_params, stage_act)):
        in_flight = min(num_mb, pp - s) if schedule == "1f1b" else num_mb
        mem.append((p * BYTES_PARAM_STATE + a * in_flight) * 1.10 / 2**30 + 2.0)
    oom = any(m > spec["mem_gb"] for m in mem)
    sc = [a + b for a, b in zip(sf, sb)]
    imb = (max(sc) - min(sc)) / max(sc) if max(sc) > 0 else 0.0
    layers = [(n - (1 if k == 0 else 0) - (1 if k == len(sizes) - 1 else 0)) / 8.0 for k, n in enumerate(sizes)]
    return Estimate(step, sf, sb, list(sizes), layers, pipe_time, max(dp_costs), tp_layer, max(opt_costs), mem, oom, num_mb, imb,
                    {"send_time": max(send) if send else 0.0})


def _estimate_hetero(model: ModelConfig, dbs: Dict[str, ProfileDB], stage_gpus: List[str], tp: int, dp: int, pp: int, mbs: int,
                     gbs: int, gpus_per_node: int, precision_bytes: int, schedule: str, sequence_parallel: bool) -> Estimate:
    if len(stage_gpus) != pp:
        raise ValueError("stage_gpus needs one GPU type per pipeline stage")
    if gbs % (dp * mbs):
        raise ValueError("gbs must be divisible by dp * mbs")
    num_mb = gbs // (dp * mbs)
    seq = model.node_sequence()
    col = {n: i for i, n in enumerate(NODE_TYPES)}
    tokens = mbs * model.seq_len
    specs = [GPU_SPECS[g] for g in stage_gpus]
    f_rows, b_rows = [], []
    for g, spec in zip(stage_gpus, specs):
        f_node, b_node = dbs[g].node_times(tp, mbs)
        f = np.array([f_node[col[n]] for n in seq])
        b = np.array([b_node[col[n]] for n in seq])
        if tp > 1:
            per_coll = spec["latency"] + (tp - 1) / tp * tokens * model.hidden * precision_bytes / spec["intra_p2p"]
            extra = 4 * per_coll * (0.35 if g == "B200" else 1.0) / 2  # only B200 has the fused TP kernels
            for i, n in enumerate(seq):
                if n in ("attn_o", "mlp_down"):
                    f[i] += extra
                    b[i] += extra
        f_rows.append(f)
        b_rows.append(b)
    world = tp * dp * pp
    inter = world > gpus_per_node and (tp * dp) >= gpus_per_node
    slow_link = min(specs, key=lambda sp: sp["inter_node"] if inter else sp["intra_p2p"])
    cut_bytes = np.array([tokens * model.cut_elems(n, tp, sequence_parallel) * precision_bytes for n in seq])
    comm = np.array([p2p_time(b, slow_link, inter) for b in cut_bytes])
    sizes = partition_hetero([f + b for f, b in zip(f_rows, b_rows)], layer_level=(tp > 1), comm=comm)
    sf, sb, stage_params, stage_act = [], [], [], []
    i = 0
    for s, n_nodes in enumerate(sizes):
        sf.append(float(f_rows[s][i:i + n_nodes].sum()))
        sb.append(float(b_rows[s][i:i + n_nodes].sum()))
        nodes = seq[i:i + n_nodes]
        stage_params.append(sum(model.node_params_sharded(n, tp) for n in nodes))
        stage_act.append(sum(model.node_act_elems(n, tp) for n in nodes) * tokens * precision_bytes)
        i += n_nodes
    bounds = np.cumsum(sizes)[:-1]
    send = []
    for k, c in enumerate(bounds):  # the link between stage k and k+1 runs at the slower side's speed
        pair = min((specs[k], specs[k + 1]), key=lambda sp: sp["inter_node"] if inter else sp["intra_p2p"])
        send.append(p2p_time(float(cut_bytes[c - 1]), pair, inter))
    ends, _ = simulate(sf, sb, send, send, num_mb, schedule)
    dp_inter = dp * tp > gpus_per_node
    dp_costs = [allreduce_time(p * 4, dp, sp, dp_inter, fused=(g == "B200")) for p, sp, g in zip(stage_params, specs, stage_gpus)]
    opt_costs = [p * 30.0 / (0.8 * sp["hbm"]) for p, sp in zip(stage_params, specs)]
    step = max(e + d + o for e, d, o in zip(ends, dp_costs, opt_costs))
    mem, oom = [], False
    for s, (p, a, sp) in enumerate(zip(stage_params, stage_act, specs)):
        in_flight = min(num_mb, pp - s) if schedule == "1f1b" else num_mb
        m = (p * BYTES_PARAM_STATE + a * in_flight) * 1.10 / 2**30 + 2.0
        mem.append(m)
        oom = oom or m > sp["mem_gb"]
    sc = [a + b for a, b in zip(sf, sb)]
    imb = (max(sc) - min(sc)) / max(sc) if max(sc) > 0 else 0.0
    layers = [(n - (1 if k == 0 else 0) - (1 if k == len(sizes) - 1 else 0)) / 8.0 for k, n in enumerate(sizes)]
    return Estimate(step, sf, sb, list(sizes), layers, max(ends), max(dp_costs), 0.0, max(opt_costs), mem, oom, num_mb, imb,
                    {"send_time": max(send) if send else 0.0, "heterogeneous": 1.0})
