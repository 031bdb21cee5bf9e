"""Continuous-batching scheduler: request queue, admission, per-step join/leave.

Absent from the reference, which serves one static batch with a fixed ``max_new_tokens`` and no early
exit (opt_prime/opt_prime/inference.py:1036).  Policy: first-come-first-served; a waiting request is
admitted when a sequence slot and enough KV pages for its prompt plus its output budget are free;
each engine step first prefills up to ``max_prefill_per_step`` admitted prompts (one forward each),
then runs one decode step for every running sequence; finished sequences release their pages at once.
The scheduler is pure host logic and is tested on CPU with a fake model.
"""
from __future__ import annotations

import collections
from dataclasses import dataclass, field
from typing import Deque, List, Optional


@dataclass
class Request:
    rid: int
    prompt: List[int]
    max_new_tokens: int
    arrival_s: float = 0.0
    eos_token_id: Optional[int] = None
    # filled while running
    slot: int = -1
    generated: List[int] = field(default_factory=list)
    t_admitted: Optional[float] = None
    t_first_token: Optional[float] = None
    t_finished: Optional[float] = None

    @property
    def prompt_len(self) -> int:
        return len(self.prompt)

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.generated)

    def is_finished(self) -> bool:
        if len(self.generated) >= self.max_new_tokens:
            return True
        return self.eos_token_id is not None and bool(self.generated) and self.generated[-1] == self.eos_token_id


@dataclass
class StepPlan:
    prefill: List[Request]
    decode: List[Request]


class ContinuousBatchingScheduler:
    def __init__(self, cache, max_running: int = 256, max_prefill_per_step: int = 4, max_prefill_tokens: int = 8192,
                 reserve_output: bool = True):
        self.cache = cache
        self.max_running = max_running
        self.max_prefill_per_step = max_prefill_per_step
        self.max_prefill_tokens = max_prefill_tokens
        self.reserve_output = reserve_output
        self.waiting: Deque[Request] = collections.deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self.peak_running = 0

    def add_request(self, req: Request) -> None:
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _budget(self, req: Request) -> int:
        return req.prompt_len + (req.max_new_tokens if self.reserve_output else 1)

    def plan_step(self, now: float) -> StepPlan:
        """Admit what fits (FCFS, no overtaking) and return this step's prefill and decode sets."""
        prefill: List[Request] = []
        tokens = 0
        while self.waiting and len(prefill) < self.max_prefill_per_step and len(self.running) + len(prefill) < self.max_running:
            req = self.waiting[0]
            if req.arrival_s > now:
                break
            if prefill and tokens + req.prompt_len > self.max_prefill_tokens:
                break
            if not self.cache.can_admit(self._budget(req)):
                break  # back-pressure: wait for pages
            self.waiting.popleft()
            req.slot = self.cache.add_sequence(self._budget(req))
            req.t_admitted = now
            prefill.append(req)
            tokens += req.prompt_len
        decode = list(self.running)
        return StepPlan(prefill, decode)

    def after_prefill(self, req: Request, first_token: int, now: float) -> None:
        req.generated.append(first_token)
        req.t_first_token = now
        self.cache.seq_len[req.slot] = req.prompt_len
        if req.is_finished():
            self._finish(req, now)
        else:
            self.running.append(req)
            self.peak_running = max(self.peak_running, len(self.running))

    def after_decode(self, reqs: List[Request], tokens: List[int], now: float) -> None:
        for req, tok in zip(reqs, tokens):
            req.generated.append(tok)
            self.cache.seq_len[req.slot] = req.total_len - 1
            if req.is_finished():
                self._finish(req, now)

    def _finish(self, req: Request, now: float) -> None:
        req.t_finished = now
        if req in self.running:
            self.running.remove(req)
        self.cache.free_sequence(req.slot)
        req.slot = -1
        self.finished.append(req)
