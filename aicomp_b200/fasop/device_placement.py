"""Heterogeneous clusters: which node type sits where along the pipeline.

A cluster is a multiset of nodes by GPU type, e.g. ``[("B200", 1), ("A100", 2)]``.  Ranks are laid out pipeline
stage by pipeline stage (``rank = stage * dp * tp + ...``), so the order of the nodes decides which stage runs on
which GPU type.  This module enumerates

* the sub-clusters worth evaluating (all of it, or every non-empty count vector for a cost/time Pareto sweep),
* the distinct orders of a multiset of node types (optionally only its cyclic rotations, which is enough when the
  pipeline is symmetric), capped so that a large cluster does not explode the search, and
* the GPU type of every pipeline stage for a given order and layout (a stage that spans two node types runs at the
  pace of the slower one).

Role of the reference's fasop/device_placement.py:14-333 (GPU type per stage, pareto cluster subsets, cyclic and
multiset permutations).
"""
from __future__ import annotations

import itertools
from typing import Dict, Iterator, List, Sequence, Tuple

from .config import GPU_SPECS

__all__ = ["cluster_subsets", "node_orders", "stage_gpu_types", "slowest"]


def cluster_subsets(gpus: Sequence[Tuple[str, int]], pareto: bool = False) -> List[List[Tuple[str, int]]]:
    """The full cluster, or (``pareto``) every sub-cluster with at least one node, largest first."""
    gpus = [(t, int(n)) for t, n in gpus if n > 0]
    if not pareto:
        return [list(gpus)]
    out = []
    for counts in itertools.product(*[range(n + 1) for _, n in gpus]):
        if sum(counts) == 0:
            continue
        out.append([(t, c) for (t, _), c in zip(gpus, counts) if c > 0])
    out.sort(key=lambda s: -sum(c for _, c in s))
    return out


def _multiset_permutations(items: List[str]) -> Iterator[Tuple[str, ...]]:
    """Distinct permutations of a multiset in lexicographic order (no duplicates are generated)."""
    a = sorted(items)
    n = len(a)
    while True:
        yield tuple(a)
        i = n - 2
        while i >= 0 and a[i] >= a[i + 1]:
            i -= 1
        if i < 0:
            return
        j = n - 1
        while a[j] <= a[i]:
            j -= 1
        a[i], a[j] = a[j], a[i]
        a[i + 1:] = reversed(a[i + 1:])


def node_orders(cluster: Sequence[Tuple[str, int]], mode: str = "permutations", limit: int = 64) -> List[Tuple[str, ...]]:
    """Orders of the nodes along the rank axis.  ``mode``: ``permutations`` (distinct orders of the multiset),
    ``cyclic`` (rotations of the grouped order) or ``grouped`` (one order, types kept together, fastest first)."""
    nodes: List[str] = []
    for t, n in sorted(cluster, key=lambda tn: -GPU_SPECS[tn[0]]["bf16_flops"]):
        nodes.extend([t] * n)
    if len(set(nodes)) <= 1 or mode == "grouped":
        return [tuple(nodes)]
    if mode == "cyclic":
        seen, out = set(), []
        for k in range(len(nodes)):
            o = tuple(nodes[k:] + nodes[:k])
            if o not in seen:
                seen.add(o)
                out.append(o)
        return out[:limit]
    if mode != "permutations":
        raise ValueError("mode must be 'permutations', 'cyclic' or 'grouped'")
    return list(itertools.islice(_multiset_permutations(nodes), limit))


def slowest(types: Sequence[str]) -> str:
    return min(types, key=lambda t: GPU_SPECS[t]["bf16_flops"])


def stage_gpu_types(order: Sequence[str], pp: int, dp: int, tp: int, gpus_per_node: int) -> List[str]:
    """GPU type of every pipeline stage when the nodes appear in ``order`` along the rank axis."""
    per_stage = dp * tp
    if pp * per_stage > len(order) * gpus_per_node:
        raise ValueError("layout needs more GPUs than the cluster has")
    out = []
    for s in range(pp):
        first, last = s * per_stage, (s + 1) * per_stage - 1
        out.append(slowest([order[n] for n in range(first // gpus_per_node, last // gpus_per_node + 1)]))
    return out


def price_per_hour(order: Sequence[str], prices: Dict[str, float]) -> float:
    return sum(prices.get(t, 0.0) for t in order)
