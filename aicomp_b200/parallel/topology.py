"""PP x DP x TP device mesh.

Rank order is the reference's (opt_prime/opt_prime/opti_pri.py:44-231):
``rank = stage * (dp * tp) + dp_idx * tp + tp_idx`` - tensor-parallel peers are
adjacent ranks (same NVSwitch domain, lowest latency for the per-layer
collectives), pipeline neighbours are ``dp * tp`` ranks apart.  Groups are
plain ``torch.distributed`` groups created collectively by every rank in the
same order; with world size 1 all groups are ``None`` and every query still
answers.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch.distributed as dist

__all__ = ["Topology"]


class Topology:
    def __init__(self, rank: int, world_size: int, pp_size: int, dp_size: int = 1, tp_size: int = 1,
                 create_groups: bool = True, backend: Optional[str] = None):
        if pp_size * dp_size * tp_size != world_size:
            raise ValueError(f"world size {world_size} != pp {pp_size} x dp {dp_size} x tp {tp_size}")
        self.rank, self.world_size = rank, world_size
        self.pp_size, self.dp_size, self.tp_size = pp_size, dp_size, tp_size
        self.num_stage = pp_size
        per_stage = dp_size * tp_size
        self.stage = rank // per_stage
        self.dp_rank = (rank // tp_size) % dp_size
        self.tp_rank = rank % tp_size
        self.stage2rank: Dict[int, List[int]] = {s: list(range(s * per_stage, (s + 1) * per_stage)) for s in range(pp_size)}
        self.tp_group = self.dp_group = self.pp_group = None
        self.fwd_groups: Dict[int, object] = {}   # boundary s -> group {rank(s), rank(s+1)} for activations
        self.bwd_groups: Dict[int, object] = {}   # same pair, separate communicator for gradients
        if create_groups and world_size > 1 and dist.is_initialized():
            self._create_groups(backend)

    # ---- rank arithmetic ------------------------------------------------
    def rank_of(self, stage: int, dp_rank: int, tp_rank: int) -> int:
        return stage * self.dp_size * self.tp_size + dp_rank * self.tp_size + tp_rank

    def tp_ranks(self, rank: Optional[int] = None) -> List[int]:
        r = self.rank if rank is None else rank
        base = r - r % self.tp_size
        return list(range(base, base + self.tp_size))

    def dp_ranks(self, rank: Optional[int] = None) -> List[int]:
        r = self.rank if rank is None else rank
        stage, tp = r // (self.dp_size * self.tp_size), r % self.tp_size
        return [self.rank_of(stage, d, tp) for d in range(self.dp_size)]

    def pp_ranks(self, rank: Optional[int] = None) -> List[int]:
        r = self.rank if rank is None else rank
        off = r % (self.dp_size * self.tp_size)
        return [s * self.dp_size * self.tp_size + off for s in range(self.pp_size)]

    def _create_groups(self, backend) -> None:
        per_stage = self.dp_size * self.tp_size
        # every rank walks all groups in the same order (new_group is collective)
        if self.tp_size > 1:
            for base in range(0, self.world_size, self.tp_size):
                ranks = list(range(base, base + self.tp_size))
                g = dist.new_group(ranks=ranks, backend=backend)
                if self.rank in ranks:
                    self.tp_group = g
        if self.dp_size > 1:
            for s in range(self.pp_size):
                for t in range(self.tp_size):
                    ranks = [self.rank_of(s, d, t) for d in range(self.dp_size)]
                    g = dist.new_group(ranks=ranks, backend=backend)
                    if self.rank in ranks:
                        self.dp_group = g
        if self.pp_size > 1:
            for off in range(per_stage):
                ranks = [s * per_stage + off for s in range(self.pp_size)]
                g = dist.new_group(ranks=ranks, backend=backend)
                if self.rank in ranks:
                    self.pp_group = g
            for s in range(self.pp_size - 1):
                for off in range(per_stage):
                    pair = [s * per_stage + off, (s + 1) * per_stage + off]
                    gf = dist.new_group(ranks=pair, backend=backend)
                    gb = dist.new_group(ranks=pair, backend=backend)
                    if self.rank in pair:
                        self.fwd_groups[s] = gf
                        self.bwd_groups[s] = gb

    # ---- queries used by the engine (names follow the reference) ----------
    def get_stage(self) -> int:
        return self.stage

    def is_first_stage(self) -> bool:
        return self.stage == 0

    def is_last_stage(self) -> bool:
        return self.stage == self.pp_size - 1

    def get_first_rank(self) -> int:
        return self.pp_ranks()[0]

    def get_last_rank(self) -> int:
        return self.pp_ranks()[-1]

    def get_prev_rank(self) -> Optional[int]:
        return None if self.is_first_stage() else self.rank - self.dp_size * self.tp_size

    def get_next_rank(self) -> Optional[int]:
        return None if self.is_last_stage() else self.rank + self.dp_size * self.tp_size

    def get_num_stage(self) -> int:
        return self.pp_size

    def __repr__(self) -> str:
        return (f"Topology(rank={self.rank}/{self.world_size}, stage={self.stage}/{self.pp_size}, "
                f"dp={self.dp_rank}/{self.dp_size}, tp={self.tp_rank}/{self.tp_size})")
