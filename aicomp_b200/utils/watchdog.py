"""Failure detection: per-rank heartbeats, step-time outliers, NaN/Inf losses, clean abort.

The reference has no failure handling in opt_prime beyond long process-group timeouts
(fasop/make_profiledb/profile_fx.py:762-771).  Here every rank publishes a heartbeat (step number and time)
in the rendezvous store from a daemon thread; any rank can ask which peers are silent.  A step that takes
``outlier_factor`` times the running median, or a loss that is not finite, is reported through the same channel.
On a detected failure the engine stops launching work, tears the process groups down and exits non-zero so the
launcher (torchrun) can restart the job from the last complete checkpoint.  Everything runs on the host:
nothing here waits on, or interrupts, a GPU.
"""
from __future__ import annotations

import math
import statistics
import threading
import time
from typing import Dict, List, Optional


class DictStore:
    """In-process stand-in for ``torch.distributed.Store`` (tests, single process)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        with self._lock:
            return self._d[key]

    def check(self, keys: List[str]) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


class Watchdog:
    def __init__(self, store, rank: int, world_size: int, interval_s: float = 1.0, timeout_s: float = 30.0, outlier_factor: float = 5.0,
                 prefix: str = "aicomp/hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval_s, self.timeout_s, self.outlier_factor = interval_s, timeout_s, outlier_factor
        self.prefix = prefix
        self.step = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._step_times: List[float] = []
        self.events: List[dict] = []
        self._paused = False

    # ---- heartbeat ---------------------------------------------------------------------------
    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self) -> None:
        self.store.set(self._key(self.rank), f"{self.step}:{time.time():.3f}")

    def _loop(self) -> None:
        while not self._stop.wait(self.interval_s):
            if not self._paused:
                try:
                    self.beat()
                except Exception:
                    return  # the store is gone: the job is going down anyway

    def start(self) -> "Watchdog":
        self.beat()
        self._thread = threading.Thread(target=self._loop, daemon=True, name="aicomp-watchdog")
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)

    def pause(self) -> None:
        """Test hook: stop beating without stopping the thread (what a wedged rank looks like from outside)."""
        self._paused = True

    def silent_ranks(self, now: Optional[float] = None) -> List[int]:
        """Ranks whose last heartbeat is older than ``timeout_s`` (or that never wrote one)."""
        now = time.time() if now is None else now
        out = []
        for r in range(self.world):
            try:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    out.append(r)
                    continue
                raw = self.store.get(self._key(r)).decode()
                t = float(raw.split(":")[1])
                if now - t > self.timeout_s:
                    out.append(r)
            except Exception:
                out.append(r)
        return out

    # ---- step health -------------------------------------------------------------------------------
    def end_step(self, step_time_s: float, loss: Optional[float] = None) -> Optional[dict]:
        """Record a finished step; returns an event dict when something is wrong, else None."""
        self.step += 1
        ev = None
        if loss is not None and not math.isfinite(loss):
            ev = {"kind": "nonfinite_loss", "step": self.step, "loss": loss}
        elif len(self._step_times) >= 5:
            med = statistics.median(self._step_times[-50:])
            if step_time_s > self.outlier_factor * med:
                ev = {"kind": "slow_step", "step": self.step, "step_time_s": step_time_s, "median_s": med}
        self._step_times.append(step_time_s)
        if ev:
            ev["rank"] = self.rank
            self.events.append(ev)
            try:
                self.store.set(f"{self.prefix}/event/{self.rank}", repr(ev))
            except Exception:
                pass
        return ev


def abort_job(reason: str, exit_code: int = 13) -> None:
    """Tear down process groups without waiting for peers and leave with a non-zero code (the launcher restarts us)."""
    import os
    import sys
    print(f"[aicomp_b200] aborting: {reason}", file=sys.stderr, flush=True)
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass
    finally:
        os._exit(exit_code)
