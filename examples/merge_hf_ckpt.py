"""CLI alias of ``python -m aicomp_b200.ckpt.merge_hf_ckpt`` under the reference's script name."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from aicomp_b200.ckpt.merge_hf_ckpt import main  # noqa: E402

if __name__ == "__main__":
    main()
