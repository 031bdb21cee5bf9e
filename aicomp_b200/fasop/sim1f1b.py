"""Event simulation of the non-interleaved 1F1B (and GPipe) schedule with asynchronous stage-to-stage transfers.

Each stage executes its operations in the order of :class:`aicomp_b200.parallel.schedule.Schedule1F1B`; a forward
of micro-batch m on stage s may start once the stage is free and the activation of (s-1, m) has arrived (end of
that forward + transfer time); backwards mirror that from the last stage.  The reference simulates the same
schedule with rendezvous (blocking) sends (fasop/stage.py:114-319); transfers here overlap compute, matching
this framework's runtime.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def stage_order(stage: int, P: int, M: int, schedule: str = "1f1b") -> List[Tuple[str, int]]:
    if schedule == "gpipe":
        return [("F", i) for i in range(M)] + [("B", i) for i in range(M)]
    warm = min(P - 1 - stage, M)
    steps = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < M:
        steps.append(("F", f)); f += 1
        steps.append(("B", b)); b += 1
    while b < M:
        steps.append(("B", b)); b += 1
    return steps


def simulate(fwd: Sequence[float], bwd: Sequence[float], send_fwd: Sequence[float], send_bwd: Sequence[float], M: int,
             schedule: str = "1f1b"):
    """Returns ``(stage_end_times, timeline)``; ``fwd/bwd`` are per-stage compute times, ``send_*[s]`` the transfer
    time across the boundary between stage s and s+1."""
    P = len(fwd)
    orders = [stage_order(s, P, M, schedule) for s in range(P)]
    ptr = [0] * P
    free_at = [0.0] * P
    f_end = [[None] * M for _ in range(P)]
    b_end = [[None] * M for _ in range(P)]
    timeline = [[] for _ in range(P)]
    remaining = sum(len(o) for o in orders)
    while remaining:
        progressed = False
        for s in range(P):
            while ptr[s] < len(orders[s]):
                kind, m = orders[s][ptr[s]]
                if kind == "F":
                    dep = 0.0 if s == 0 else (None if f_end[s - 1][m] is None else f_end[s - 1][m] + send_fwd[s - 1])
                else:
                    if s == P - 1:
                        dep = f_end[s][m]
                    else:
                        dep = None if b_end[s + 1][m] is None else b_end[s + 1][m] + send_bwd[s]
                if dep is None:
                    break
                start = max(free_at[s], dep)
                end = start + (fwd[s] if kind == "F" else bwd[s])
                (f_end if kind == "F" else b_end)[s][m] = end
                free_at[s] = end
                timeline[s].append((kind, m, start, end))
                ptr[s] += 1
                remaining -= 1
                progressed = True
        if not progressed:
            raise RuntimeError("pipeline simulation deadlocked (inconsistent schedule)")
    return free_at, timeline


def bubble_fraction(fwd, bwd, M: int) -> float:
    P = len(fwd)
    end, _ = simulate(fwd, bwd, [0.0] * (P - 1), [0.0] * (P - 1), M)
    busy = max(M * (f + b) for f, b in zip(fwd, bwd))
    return 1.0 - busy / max(end) if max(end) > 0 else 0.0
