"""Pipeline partitioners: node -> stage assignment on a traced module-level graph.

Methods (names as in the reference, opt_prime/opt_prime/IR.py:1747-1799):

``simple``          cut after every ``modcnt // num_stage`` ``call_module`` nodes
                    (IR.py:1803-1966); the last stage takes the remainder.
``llama-tp-split``  cut only at decoder-layer boundaries, blocks = embedding +
                    layers + head spread evenly (IR.py:2541-2726).
``milp``            minimise bytes crossing stage boundaries under memory and
                    node-count balance, solved with HiGHS through
                    ``scipy.optimize.milp`` (capability of IR.py:1969-2216).
``hierarchical``    the same program on block-level super-nodes, for graphs
                    with thousands of modules such as MoE models
                    (IR.py:2219-2538); imbalance bounds overridable through
                    ``OPT_PRIME_HIER_COUNT_IMBALANCE`` / ``OPT_PRIME_HIER_MEM_IMBALANCE``.

The integer program here is a chain formulation of our own: units are ordered
as in the graph, ``x[i,k]`` puts unit ``i`` on stage ``k``, the stage index
``s_i = sum_k k x[i,k]`` may only stay or step by one along the chain, and the
objective ``sum_c W_c (s_{c+1} - s_c)`` charges every cut ``c`` with the bytes
of all values that are live across it (a value relayed over several stages is
charged once per hop, which is what the runtime does).  All assignments are
O(N) or one small MILP; any solver failure falls back to ``simple``.
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Optional, Tuple

import torch
import torch.fx as fx

from ..utils.log import get_logger

log = get_logger(__name__)

__all__ = ["assign_stages", "PARTITIONERS", "block_index_of"]

PARTITIONERS = ("auto", "simple", "milp", "hierarchical", "llama-tp-split", "balanced")

_BLOCK_RE = re.compile(r"(?:^|[._])(?:layers|h|layer|blocks|block)[._](\d+)(?:[._]|$)")


def block_index_of(target: str) -> Optional[int]:
    """Index of the repeated block a module path belongs to (``model.layers.3.mlp`` -> 3)."""
    m = _BLOCK_RE.search(target)
    return int(m.group(1)) if m else None


def _compute_nodes(gm: fx.GraphModule) -> List[fx.Node]:
    return [n for n in gm.graph.nodes if n.op not in ("placeholder", "output")]


def _finalise(gm: fx.GraphModule, stage_of_compute: Dict[fx.Node, int], num_stage: int) -> Dict[fx.Node, int]:
    """Placeholders live on stage 0, the output node on the last stage; stages are made monotone in node order."""
    out: Dict[fx.Node, int] = {}
    cur = 0
    for n in gm.graph.nodes:
        if n.op == "placeholder":
            out[n] = 0
        elif n.op == "output":
            out[n] = num_stage - 1
        else:
            cur = max(cur, stage_of_compute[n])
            out[n] = min(cur, num_stage - 1)
    # get_attr nodes follow their first user so parameters land where they are consumed
    for n in gm.graph.nodes:
        if n.op == "get_attr" and n.users:
            out[n] = min(out[u] for u in n.users)
    return out


def assign_simple(gm: fx.GraphModule, num_stage: int) -> Dict[fx.Node, int]:
    nodes = _compute_nodes(gm)
    modcnt = sum(1 for n in nodes if n.op == "call_module")
    if modcnt < num_stage:
        raise ValueError(f"model has {modcnt} modules, fewer than {num_stage} stages")
    segment = modcnt // num_stage
    stage, cnt = 0, 0
    res: Dict[fx.Node, int] = {}
    for n in nodes:
        res[n] = stage
        if n.op == "call_module":
            cnt += 1
            if cnt == segment and stage < num_stage - 1:
                stage += 1
                cnt = 0
    return _finalise(gm, res, num_stage)


def _block_of_nodes(gm: fx.GraphModule) -> Tuple[List[fx.Node], List[int], int]:
    """Map every compute node to a block id: 0 = pre-layer part, 1..L = layers, L+1 = head."""
    nodes = _compute_nodes(gm)
    raw: List[Optional[int]] = [block_index_of(str(n.target)) if n.op in ("call_module", "get_attr") else None for n in nodes]
    layer_ids = sorted({r for r in raw if r is not None})
    if not layer_ids:
        raise ValueError("no repeated layer blocks found in the graph")
    first_pos = {l: min(i for i, r in enumerate(raw) if r == l) for l in layer_ids}
    starts = sorted((first_pos[l], l) for l in layer_ids)
    # a layer's region starts at the first node whose inputs only that layer consumes; approximated by the first
    # module node of the layer, moved back over the shape/getattr glue that directly precedes it
    blocks: List[int] = [0] * len(nodes)
    last_layer_end = max(i for i, r in enumerate(raw) if r is not None)
    cur = 0
    start_idx = {pos: k + 1 for k, (pos, _) in enumerate(starts)}
    for i in range(len(nodes)):
        if i in start_idx:
            cur = start_idx[i]
        blocks[i] = cur
    n_layers = len(layer_ids)
    # nodes after the last layer module that do not belong to it form the head block; the residual add that
    # closes the last layer stays with the layer (everything up to the next call_module)
    j = last_layer_end + 1
    while j < len(nodes) and nodes[j].op != "call_module":
        j += 1
    for i in range(j, len(nodes)):
        blocks[i] = n_layers + 1
    return nodes, blocks, n_layers


def assign_llama_tp_split(gm: fx.GraphModule, num_stage: int) -> Dict[fx.Node, int]:
    nodes, blocks, n_layers = _block_of_nodes(gm)
    num_blocks = n_layers + 2
    if num_blocks < num_stage:
        raise ValueError(f"{num_blocks} blocks cannot fill {num_stage} stages")
    bounds = [(i * num_blocks) // num_stage for i in range(num_stage + 1)]
    # the head block is heavy (vocab projection): when the last two stages would be uneven, give the last one less
    if num_stage >= 2 and (bounds[-1] - bounds[-2]) > (bounds[-2] - bounds[-3]):
        bounds[-2] += 1
    stage_of_block = {}
    for s in range(num_stage):
        for b in range(bounds[s], bounds[s + 1]):
            stage_of_block[b] = s
    res = {n: stage_of_block[b] for n, b in zip(nodes, blocks)}
    return _finalise(gm, res, num_stage)


def assign_balanced(gm: fx.GraphModule, num_stage: int) -> Dict[fx.Node, int]:
    """Contiguous split that minimises the heaviest stage, with a module's matmul parameter count as its cost.

    For transformer stacks the FLOPs of a module are proportional to the parameters it multiplies with, so this
    balances compute: the vocabulary projection counts as ~2.4 Llama-3-8B layers, the embedding lookup as nothing.
    Exact dynamic programme over the positions after each ``call_module``.  Not in the reference, whose ``simple``
    split counts modules (IR.py:1803-1966) and leaves the last stage with the head on top of an equal layer share.
    """
    nodes = _compute_nodes(gm)
    mod_pos = [i for i, n in enumerate(nodes) if n.op == "call_module"]
    if len(mod_pos) < num_stage:
        raise ValueError("fewer modules than stages")
    w = []
    for i in mod_pos:
        m = gm.get_submodule(str(nodes[i].target))
        if "embedding" in type(m).__name__.lower():
            w.append(0.0)
        else:
            w.append(float(sum(p.numel() for p in m.parameters() if p.dim() >= 2)) + 1.0)
    n = len(w)
    pre = [0.0]
    for x in w:
        pre.append(pre[-1] + x)
    INF = float("inf")
    best = [[INF] * (n + 1) for _ in range(num_stage + 1)]
    back = [[0] * (n + 1) for _ in range(num_stage + 1)]
    best[0][0] = 0.0
    for s in range(1, num_stage + 1):
        for j in range(s, n + 1):
            for i in range(s - 1, j):
                if best[s - 1][i] == INF:
                    continue
                v = max(best[s - 1][i], pre[j] - pre[i])
                if v < best[s][j]:
                    best[s][j], back[s][j] = v, i
    cuts, j = [], n
    for s in range(num_stage, 0, -1):
        cuts.append(j)
        j = back[s][j]
    cuts = cuts[::-1]  # number of modules up to and including each stage
    stage_of_mod = []
    s = 0
    for k in range(n):
        while k >= cuts[s]:
            s += 1
        stage_of_mod.append(s)
    res: Dict[fx.Node, int] = {}
    cur, k = 0, 0
    for i, node in enumerate(nodes):
        if node.op == "call_module":
            cur = stage_of_mod[k]
            k += 1
        res[node] = cur
    # glue that follows a stage's last module (e.g. the residual add) stays with it: nodes take the stage of the
    # most recent module, so only the glue BEFORE the first module of a stage needs pulling back
    return _finalise(gm, res, num_stage)


# ------------------------------------------------------------------ MILP on a chain of units
def _bytes_of(meta) -> int:
    if meta is None:
        return 0
    shape, dtype = meta
    n = 1
    for d in shape:
        n *= int(d)
    return n * torch.empty((), dtype=dtype).element_size()


def _module_bytes(gm: fx.GraphModule, node: fx.Node) -> int:
    if node.op == "call_module":
        try:
            m = gm.get_submodule(str(node.target))
        except AttributeError:
            return 0
        return sum(p.numel() * p.element_size() for p in m.parameters()) + sum(b.numel() * b.element_size() for b in m.buffers())
    if node.op == "get_attr":
        obj = gm
        try:
            for part in str(node.target).split("."):
                obj = getattr(obj, part)
        except AttributeError:
            return 0
        if isinstance(obj, torch.Tensor):
            return obj.numel() * obj.element_size()
    return 0


def _units(gm: fx.GraphModule, hierarchical: bool) -> Tuple[List[fx.Node], List[int]]:
    """Group compute nodes into chain units: one per call_module (plus trailing glue), or one per block."""
    nodes = _compute_nodes(gm)
    unit_of: List[int] = []
    if hierarchical:
        try:
            _, blocks, _ = _block_of_nodes(gm)
            return nodes, blocks
        except ValueError:
            pass
    u = -1
    for n in nodes:
        if n.op == "call_module" or u < 0:
            u += 1
        unit_of.append(u)
    return nodes, unit_of


def _solve_chain_milp(mem: List[float], cnt: List[int], cut_w: List[float], K: int, mem_imb: float, cnt_imb: float,
                      time_limit: float = 30.0) -> Optional[List[int]]:
    import numpy as np
    from scipy.optimize import Bounds, LinearConstraint, milp
    from scipy.sparse import lil_matrix

    n = len(mem)
    if n < K:
        return None
    nv = n * K

    def var(i, k):
        return i * K + k

    # objective: sum_c W_c (s_{c+1} - s_c), s_i = sum_k k x[i,k]
    c = np.zeros(nv)
    for cpos, w in enumerate(cut_w):
        for k in range(K):
            c[var(cpos + 1, k)] += w * k
            c[var(cpos, k)] -= w * k
    rows = []
    lo, hi = [], []
    A = lil_matrix((n + 2 * (n - 1) + 2 * K + 2, nv))
    r = 0
    for i in range(n):  # one stage per unit
        for k in range(K):
            A[r, var(i, k)] = 1
        lo.append(1); hi.append(1); r += 1
    for i in range(n - 1):  # 0 <= s_{i+1} - s_i <= 1
        for k in range(K):
            A[r, var(i + 1, k)] = k
            A[r, var(i, k)] = -k
        lo.append(0); hi.append(1); r += 1
    total_mem, total_cnt = sum(mem), sum(cnt)
    mem_cap = max(mem_imb * total_mem / K, 1.05 * max(mem)) if total_mem > 0 else float("inf")
    for k in range(K):  # memory and count balance per stage
        for i in range(n):
            A[r, var(i, k)] = mem[i]
        lo.append(0); hi.append(mem_cap if np.isfinite(mem_cap) else 1e30); r += 1
    cnt_lo, cnt_hi = total_cnt / K / cnt_imb, total_cnt / K * cnt_imb
    for k in range(K):
        for i in range(n):
            A[r, var(i, k)] = cnt[i]
        lo.append(min(cnt_lo, total_cnt / K)); hi.append(max(cnt_hi, max(cnt))); r += 1
    A[r, var(0, 0)] = 1; lo.append(1); hi.append(1); r += 1           # first unit on stage 0
    A[r, var(n - 1, K - 1)] = 1; lo.append(1); hi.append(1); r += 1   # last unit on the last stage
    A = A.tocsr()[:r]
    try:
        res = milp(c, constraints=LinearConstraint(A, np.array(lo), np.array(hi)), integrality=np.ones(nv),
                   bounds=Bounds(0, 1), options={"time_limit": time_limit, "mip_rel_gap": 0.05, "disp": False})
    except Exception as e:  # solver unavailable / numerical trouble
        log.warning("chain MILP failed: %r", e)
        return None
    if res.x is None:
        return None
    x = res.x.reshape(n, K)
    stages = [int(x[i].argmax()) for i in range(n)]
    for i in range(1, n):  # monotone repair against rounding noise
        stages[i] = max(stages[i], stages[i - 1])
    return stages


def _assign_milp(gm: fx.GraphModule, num_stage: int, hierarchical: bool) -> Dict[fx.Node, int]:
    nodes, unit_of = _units(gm, hierarchical)
    n_units = max(unit_of) + 1
    if n_units < num_stage:
        raise ValueError("fewer partition units than stages")
    mem = [0.0] * n_units
    cnt = [0] * n_units
    pos = {n: u for n, u in zip(nodes, unit_of)}
    for n, u in zip(nodes, unit_of):
        mem[u] += _module_bytes(gm, n)
        cnt[u] += 1 if n.op == "call_module" else 0
    cut_w = [0.0] * (n_units - 1)
    for n in nodes:
        if not n.users:
            continue
        last = max((pos[u] for u in n.users if u in pos), default=pos[n])
        b = float(_bytes_of(n.meta.get("tensor_meta"))) or 8.0
        for cpos in range(pos[n], last):
            cut_w[cpos] += b
    if hierarchical:
        cnt_imb = float(os.environ.get("OPT_PRIME_HIER_COUNT_IMBALANCE", "1.5"))
        mem_imb = float(os.environ.get("OPT_PRIME_HIER_MEM_IMBALANCE", "1.5"))
    else:
        cnt_imb, mem_imb = 1.3, 1.5
    stages = _solve_chain_milp(mem, cnt, cut_w, num_stage, mem_imb, cnt_imb)
    if stages is None or len(set(stages)) < num_stage:
        log.warning("MILP partition infeasible or incomplete; falling back to 'simple'")
        return assign_simple(gm, num_stage)
    res = {n: stages[u] for n, u in zip(nodes, unit_of)}
    return _finalise(gm, res, num_stage)


def assign_stages(gm: fx.GraphModule, num_stage: int, method: str = "auto", is_llama: bool = False, tp_size: int = 1
                  ) -> Dict[fx.Node, int]:
    """Return ``{node: stage}`` for every node of ``gm``; ``auto`` picks ``llama-tp-split`` for Llama with TP."""
    if method not in PARTITIONERS:
        raise ValueError(f"partitioner must be one of {PARTITIONERS}")
    if num_stage == 1:
        return {n: 0 for n in gm.graph.nodes}
    if method == "auto":
        fused_layers = any(n.op == "call_module" and type(gm.get_submodule(str(n.target))).__name__ == "B200LlamaLayer"
                           for n in gm.graph.nodes)
        method = "llama-tp-split" if (is_llama and tp_size > 1 and not fused_layers) else ("balanced" if fused_layers else "simple")
    if is_llama and tp_size > 1 and method not in ("llama-tp-split", "balanced"):
        log.warning("Llama with tensor parallelism uses the 'llama-tp-split' partitioner (was %s)", method)
        method = "llama-tp-split"
    if method == "simple":
        return assign_simple(gm, num_stage)
    if method == "balanced":
        return assign_balanced(gm, num_stage)
    if method == "llama-tp-split":
        try:
            return assign_llama_tp_split(gm, num_stage)
        except ValueError as e:
            log.warning("llama-tp-split not applicable (%s); using 'simple'", e)
            return assign_simple(gm, num_stage)
    return _assign_milp(gm, num_stage, hierarchical=(method == "hierarchical"))
