"""Pipeline partitioners over a sequence of node costs (which nodes go to which stage, contiguous).

Methods of the reference (fasop/pipe.py:78-1185): ``minmax`` (greedy move of one boundary node from the heaviest
to a lighter neighbour until no move helps), ``dp`` (dynamic programme minimising the largest stage),
``ilp`` (integer programme: here HiGHS through ``scipy.optimize.milp``, since OR-tools is optional), ``bruteforce``
(all compositions, small problems only) and ``optimus-even`` (the split the training engine itself would make:
even in layers, see :mod:`aicomp_b200.graph.partition`).  With TP > 1 cuts are restricted to layer boundaries.
Each returns the list of stage sizes (number of nodes per stage).
"""
from __future__ import annotations

import itertools
from typing import List, Optional, Sequence

import numpy as np

NODES_PER_LAYER = 8


def stage_costs(cost: Sequence[float], sizes: Sequence[int]) -> List[float]:
    out, i = [], 0
    for n in sizes:
        out.append(float(sum(cost[i:i + n])))
        i += n
    return out


def _allowed_cuts(n_nodes: int, layer_level: bool) -> List[int]:
    """Positions c (1..n-1) where a cut may be placed (a cut at c separates nodes [..c-1] | [c..])."""
    if not layer_level:
        return list(range(1, n_nodes))
    # node 0 is the embedding, then layers of 8 nodes, then lm_head
    return [1 + NODES_PER_LAYER * k for k in range(0, (n_nodes - 2) // NODES_PER_LAYER + 1) if 0 < 1 + NODES_PER_LAYER * k < n_nodes]


def partition_even(n_nodes: int, pp: int, layer_level: bool = True) -> List[int]:
    """What the engine's own splitter does: embedding + layers + head as blocks, spread evenly over the stages."""
    n_layers = (n_nodes - 2) // NODES_PER_LAYER
    blocks = n_layers + 2
    bounds = [(i * blocks) // pp for i in range(pp + 1)]
    if pp >= 2 and (bounds[-1] - bounds[-2]) > (bounds[-2] - bounds[-3]):
        bounds[-2] += 1
    sizes = []
    for s in range(pp):
        n = 0
        for b in range(bounds[s], bounds[s + 1]):
            n += 1 if b in (0, blocks - 1) else NODES_PER_LAYER
        sizes.append(n)
    return sizes


def partition_dp(cost: Sequence[float], pp: int, layer_level: bool = False, comm: Optional[Sequence[float]] = None) -> List[int]:
    """Minimise the maximum stage cost (compute plus the transfer across the stage's outgoing cut)."""
    n = len(cost)
    cuts = [0] + _allowed_cuts(n, layer_level) + [n]
    idx = {c: i for i, c in enumerate(cuts)}
    pre = np.concatenate([[0.0], np.cumsum(cost)])
    INF = float("inf")
    K = len(cuts)
    best = [[INF] * K for _ in range(pp + 1)]
    back = [[-1] * K for _ in range(pp + 1)]
    best[0][0] = 0.0
    for s in range(1, pp + 1):
        for j in range(1, K):
            for i in range(j):
                if best[s - 1][i] == INF:
                    continue
                seg = pre[cuts[j]] - pre[cuts[i]]
                if comm is not None and cuts[j] < n:
                    seg += comm[cuts[j] - 1]
                v = max(best[s - 1][i], seg)
                if v < best[s][j]:
                    best[s][j], back[s][j] = v, i
    if best[pp][K - 1] == INF:
        raise ValueError("no feasible partition")
    sizes, j = [], K - 1
    for s in range(pp, 0, -1):
        i = back[s][j]
        sizes.append(cuts[j] - cuts[i])
        j = i
    return sizes[::-1]


def partition_hetero(cost_by_stage: Sequence[Sequence[float]], layer_level: bool = False,
                     comm: Optional[Sequence[float]] = None) -> List[int]:
    """Minimise the maximum stage cost when stage ``s`` pays ``cost_by_stage[s][node]`` for a node (stages on
    different GPU types): the same dynamic programme as :func:`partition_dp` with one prefix sum per stage."""
    pp = len(cost_by_stage)
    n = len(cost_by_stage[0])
    cuts = [0] + _allowed_cuts(n, layer_level) + [n]
    pre = [np.concatenate([[0.0], np.cumsum(c)]) for c in cost_by_stage]
    INF = float("inf")
    K = len(cuts)
    best = [[INF] * K for _ in range(pp + 1)]
    back = [[-1] * K for _ in range(pp + 1)]
    best[0][0] = 0.0
    for s in range(1, pp + 1):
        ps = pre[s - 1]
        for j in range(1, K):
            for i in range(j):
                if best[s - 1][i] == INF:
                    continue
                seg = ps[cuts[j]] - ps[cuts[i]]
                if comm is not None and cuts[j] < n:
                    seg += comm[cuts[j] - 1]
                v = max(best[s - 1][i], seg)
                if v < best[s][j]:
                    best[s][j], back[s][j] = v, i
    if best[pp][K - 1] == INF:
        raise ValueError("no feasible partition")
    sizes, j = [], K - 1
    for s in range(pp, 0, -1):
        i = back[s][j]
        sizes.append(cuts[j] - cuts[i])
        j = i
    return sizes[::-1]


def partition_minmax(cost: Sequence[float], pp: int, layer_level: bool = False, max_iter: int = 10000) -> List[int]:
    """Greedy boundary shifting: move one node (or one layer) across a stage boundary whenever that lowers the larger
    of the two stages it separates; stop when no boundary can be improved (or a state repeats)."""
    n = len(cost)
    if layer_level and (n - 2) % NODES_PER_LAYER == 0:
        sizes = partition_even(n, pp)
    else:
        sizes = [n // pp + (1 if i < n % pp else 0) for i in range(pp)]
    step = NODES_PER_LAYER if layer_level else 1
    pre = np.concatenate([[0.0], np.cumsum(cost)])
    seen = set()
    for _ in range(max_iter):
        key = tuple(sizes)
        if key in seen:
            break
        seen.add(key)
        improved = False
        bounds = np.concatenate([[0], np.cumsum(sizes)]).astype(int)
        for b in range(1, pp):  # boundary between stage b-1 and b
            left = pre[bounds[b]] - pre[bounds[b - 1]]
            right = pre[bounds[b + 1]] - pre[bounds[b]]
            cur = max(left, right)
            for d in (-step, step):
                nb = bounds[b] + d
                if nb <= bounds[b - 1] or nb >= bounds[b + 1]:
                    continue
                trial = list(sizes)
                trial[b - 1] += d
                trial[b] -= d
                if layer_level and not _valid_layer_sizes(trial, n):
                    continue
                l2, r2 = pre[nb] - pre[bounds[b - 1]], pre[bounds[b + 1]] - pre[nb]
                if max(l2, r2) < cur - 1e-15:
                    sizes, improved = trial, True
                    break
            if improved:
                break
        if not improved:
            break
    return sizes


def _valid_layer_sizes(sizes: Sequence[int], n: int) -> bool:
    allowed = set(_allowed_cuts(n, True))
    c = 0
    for s in sizes[:-1]:
        c += s
        if c not in allowed:
            return False
    return all(s >= 1 for s in sizes)


def partition_bruteforce(cost: Sequence[float], pp: int, layer_level: bool = False, limit: int = 2_000_000) -> List[int]:
    n = len(cost)
    cuts = _allowed_cuts(n, layer_level)
    best, best_sizes, count = float("inf"), None, 0
    for combo in itertools.combinations(cuts, pp - 1):
        count += 1
        if count > limit:
            break
        b = (0,) + combo + (n,)
        sizes = [b[i + 1] - b[i] for i in range(pp)]
        v = max(stage_costs(cost, sizes))
        if v < best:
            best, best_sizes = v, sizes
    if best_sizes is None:
        raise ValueError("no feasible partition")
    return best_sizes


def partition_ilp(cost: Sequence[float], pp: int, layer_level: bool = False, num_mb: int = 1, time_limit: float = 30.0) -> List[int]:
    """minimise (num_mb - 1) * T + sum_s stage_s  s.t.  T >= stage_s, contiguous stages (chain formulation)."""
    from scipy.optimize import Bounds, LinearConstraint, milp
    from scipy.sparse import lil_matrix
    n = len(cost)
    cuts = [0] + _allowed_cuts(n, layer_level) + [n]
    units = [float(sum(cost[cuts[i]:cuts[i + 1]])) for i in range(len(cuts) - 1)]
    U = len(units)
    if U < pp:
        raise ValueError("fewer units than stages")
    nv = U * pp + 1
    T = nv - 1

    def var(i, k):
        return i * pp + k
    c = np.zeros(nv)
    c[T] = max(num_mb - 1, 1)
    rows, lo, hi = [], [], []
    A = lil_matrix((U + (U - 1) + pp + 2, nv))
    r = 0
    for i in range(U):
        for k in range(pp):
            A[r, var(i, k)] = 1
        lo.append(1); hi.append(1); r += 1
    for i in range(U - 1):
        for k in range(pp):
            A[r, var(i + 1, k)] = k
            A[r, var(i, k)] = -k
        lo.append(0); hi.append(1); r += 1
    for k in range(pp):
        for i in range(U):
            A[r, var(i, k)] = units[i]
        A[r, T] = -1
        lo.append(-np.inf); hi.append(0); r += 1
    A[r, var(0, 0)] = 1; lo.append(1); hi.append(1); r += 1
    A[r, var(U - 1, pp - 1)] = 1; lo.append(1); hi.append(1); r += 1
    integrality = np.ones(nv); integrality[T] = 0
    ub = np.ones(nv); ub[T] = np.inf
    res = milp(c, constraints=LinearConstraint(A.tocsr()[:r], np.array(lo), np.array(hi)), integrality=integrality,
               bounds=Bounds(np.zeros(nv), ub), options={"time_limit": time_limit, "disp": False})
    if res.x is None:
        raise RuntimeError("ILP found no solution")
    x = res.x[:-1].reshape(U, pp)
    stage = [int(x[i].argmax()) for i in range(U)]
    for i in range(1, U):
        stage[i] = max(stage[i], stage[i - 1])
    sizes = [0] * pp
    for i, s in enumerate(stage):
        sizes[s] += cuts[i + 1] - cuts[i]
    return sizes


PARTITION_METHODS = ("minmax", "optimus-even", "dp", "ilp", "bruteforce")


def partition(method: str, cost: Sequence[float], pp: int, layer_level: bool, num_mb: int = 1,
              comm: Optional[Sequence[float]] = None) -> List[int]:
    if pp == 1:
        return [len(cost)]
    if method == "optimus-even":
        return partition_even(len(cost), pp)
    if method == "minmax":
        return partition_minmax(cost, pp, layer_level)
    if method == "dp":
        return partition_dp(cost, pp, layer_level, comm)
    if method == "ilp":
        try:
            return partition_ilp(cost, pp, layer_level, num_mb)
        except Exception:
            return partition_dp(cost, pp, layer_level, comm)
    if method == "bruteforce":
        return partition_bruteforce(cost, pp, layer_level)
    raise ValueError(f"unknown partition method {method}")
