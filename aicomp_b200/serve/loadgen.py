"""Synthetic serving load and metrics (Poisson arrivals, uniform prompt/output lengths, TTFT / throughput)."""
from __future__ import annotations

import random
from typing import Dict, List

from .scheduler import Request


def make_requests(n: int, rate_per_s: float, prompt_range=(128, 2048), output_range=(64, 512), vocab: int = 128256, seed: int = 0
                  ) -> List[Request]:
    """``n`` requests with exponential inter-arrival times (rate ``rate_per_s``) and uniform lengths / token ids."""
    rng = random.Random(seed)
    t = 0.0
    reqs = []
    for i in range(n):
        t += rng.expovariate(rate_per_s) if rate_per_s > 0 else 0.0
        plen = rng.randint(*prompt_range)
        olen = rng.randint(*output_range)
        prompt = [rng.randrange(vocab) for _ in range(plen)]
        reqs.append(Request(rid=i, prompt=prompt, max_new_tokens=olen, arrival_s=t))
    return reqs


def percentile(values: List[float], q: float) -> float:
    if not values:
        return float("nan")
    s = sorted(values)
    k = (len(s) - 1) * q
    lo, hi = int(k), min(int(k) + 1, len(s) - 1)
    return s[lo] + (s[hi] - s[lo]) * (k - lo)


def summarize(finished: List[Request], wall_s: float) -> Dict[str, float]:
    ttft = [r.t_first_token - r.arrival_s for r in finished if r.t_first_token is not None]
    out_tokens = sum(len(r.generated) for r in finished)
    decode_tokens = sum(max(0, len(r.generated) - 1) for r in finished)
    e2e = [r.t_finished - r.arrival_s for r in finished if r.t_finished is not None]
    tpot = [(r.t_finished - r.t_first_token) / max(1, len(r.generated) - 1) for r in finished
            if r.t_finished is not None and r.t_first_token is not None and len(r.generated) > 1]
    return {
        "requests": len(finished), "wall_s": wall_s, "output_tokens": out_tokens,
        "decode_tokens_per_s": decode_tokens / wall_s if wall_s > 0 else float("nan"),
        "output_tokens_per_s": out_tokens / wall_s if wall_s > 0 else float("nan"),
        "ttft_p50_s": percentile(ttft, 0.5), "ttft_p99_s": percentile(ttft, 0.99),
        "tpot_p50_s": percentile(tpot, 0.5), "e2e_p50_s": percentile(e2e, 0.5),
    }
