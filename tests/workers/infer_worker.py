"""Rank body: generation through Optimus_Inference on gloo ranks."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from tests.dist_utils import worker_args, worker_report  # noqa: E402
from tests.models_small import build_model  # noqa: E402

from aicomp_b200 import Optimus_Inference  # noqa: E402


def main():
    a = worker_args()
    eng = Optimus_Inference(build_model("llama"), use_gpu=False, pp_size=a["pp"], tp_size=a["tp"], use_kv_cache=a["kv"],
                            max_seq_len=64, dtype=torch.float32)
    ids = torch.tensor([[5, 7, 11, 13], [2, 3, 4, 9]]) if eng.is_first_stage() else None
    out = eng.generate(ids, max_new_tokens=a["new"], do_sample=False, verbose=False)
    worker_report({"ids": out.tolist() if out is not None else None})
    eng.barrier()


if __name__ == "__main__":
    main()
