"""Rank body: continuous-batching serving on a tensor-parallel replica (gloo ranks, real-time arrivals)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from tests.dist_utils import worker_args, worker_report  # noqa: E402
from tests.models_small import build_model  # noqa: E402

from aicomp_b200.serve.engine import ServingEngine  # noqa: E402
from aicomp_b200.serve.scheduler import Request  # noqa: E402


def main():
    a = worker_args()
    torch.manual_seed(0)
    eng = ServingEngine(build_model("llama"), tp_size=a["tp"], use_gpu=False, num_pages=64, max_seqs=4, max_seq_len=64,
                        dtype=torch.float32)
    prompts = [[5, 7, 11, 13, 17], [2, 3], [9] * 19, [1, 2, 3, 4, 5, 6, 7], [8, 8, 8], [3, 1, 4, 1, 5, 9, 2, 6]]
    news = [6, 9, 4, 12, 5, 7]
    # arrivals a few milliseconds apart: ranks whose clocks disagree by microseconds would admit them in different steps
    reqs = [Request(rid=i, prompt=p, max_new_tokens=n, arrival_s=0.004 * i) for i, (p, n) in enumerate(zip(prompts, news))]
    m = eng.serve(reqs, realtime=True)
    got = {r.rid: r.generated for r in eng.scheduler.finished}
    worker_report({"tokens": [got[i] for i in range(len(prompts))], "requests": m["requests"], "unfinished": m["unfinished"]})
    eng.comm.barrier()


if __name__ == "__main__":
    main()
