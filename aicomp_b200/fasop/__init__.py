"""FASOP for B200: strategy search over PP x TP x DP x micro-batch with a profile-driven cost model.

Capabilities of the reference's ``fasop/`` tree (FASOP.py, config.py, estimate.py, pipe.py, stage.py, partition.py,
device_placement.py, utils.py, make_profiledb/), rebuilt around B200 measurements: NVSwitch alpha-beta
communication model instead of A40/PCIe tiers, SwiGLU/GQA-correct parameter and activation counts, separate
forward and backward node costs, per-stage data-parallel cost, and an event simulation of the 1F1B schedule this
framework actually runs (asynchronous sends).  ``python -m aicomp_b200.fasop --gpus B200 8 --model-type llama3b ...``.
"""
from .config import MODEL_CONFIGS, NODE_TYPES, ModelConfig, GPU_SPECS  # noqa: F401
from .search import FasopConfig, SearchResult, run_strategy_search  # noqa: F401
