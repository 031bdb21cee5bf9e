"""Pareto output: JSON always, a PNG when matplotlib is installed (the reference plots with matplotlib, fasop/utils.py:262-378)."""
from __future__ import annotations

import json
from dataclasses import asdict
from typing import List


def save_pareto(front: List, stem: str, title: str = "FASOP") -> str:
    with open(stem + ".json", "w") as f:
        json.dump([asdict(r) for r in front], f, indent=1)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        return stem + ".json"
    fig, ax = plt.subplots(figsize=(6, 4))
    ax.plot([r.total_time / 3600 for r in front], [r.cost for r in front], "o-")
    for r in front:
        ax.annotate(f"tp{r.tp} dp{r.dp} pp{r.pp} mbs{r.mbs}", (r.total_time / 3600, r.cost), fontsize=6)
    ax.set_xlabel("total time (h)")
    ax.set_ylabel("cost ($)")
    ax.set_title(title)
    fig.savefig(stem + ".png", dpi=150, bbox_inches="tight")
    return stem + ".png"
