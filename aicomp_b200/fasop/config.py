"""Static tables of the cost model: hardware, prices, datasets, model shapes, per-node parameter/activation counts.

Node types are the reference's ten FX node kinds (fasop/config.py:281-302) so that profile databases stay
interchangeable: ``embed, attn_q, attn_k, attn_v, attn_o, mlp_gate, mlp_act_fn, mlp_up, mlp_down, lm_head``.
Parameter and activation formulas use the real FFN width and GQA head counts (the reference assumes FFN = 4h,
fasop/config.py:371-374).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

NODE_TYPES = ("embed", "attn_q", "attn_k", "attn_v", "attn_o", "mlp_gate", "mlp_act_fn", "mlp_up", "mlp_down", "lm_head")
LAYER_NODES = NODE_TYPES[1:9]
MBS_OPTIONS = (1, 2, 4, 8, 16, 32, 64, 128)

# Bandwidths in bytes/s, latencies in seconds.  B200 numbers: NVLink 5 through NVSwitch, uniform to every peer;
# all-reduce bus bandwidth and peer-copy bandwidth are the values measured on an 8 x B200 box, `fused_*` are this
# framework's peer-memory kernels.  A40/A100/A10 rows keep the reference's constants (fasop/config.py:17-59).
GPU_SPECS: Dict[str, Dict[str, float]] = {
    "B200": {"mem_gb": 180.0, "intra_p2p": 770e9, "intra_allreduce_bus": 725e9, "fused_allreduce_bus": 629e9,
             "inter_node": 400e9 / 8, "latency": 8e-6, "hbm": 6.5e12, "bf16_flops": 1.4e15},
    "A100": {"mem_gb": 39.59, "intra_p2p": 300e9, "intra_allreduce_bus": 230e9, "inter_node": 40e9 / 8, "latency": 15e-6,
             "hbm": 1.5e12, "bf16_flops": 2.5e14},
    "A40": {"mem_gb": 47.0, "intra_p2p": 46.89e9, "intra_allreduce_bus": 43.94e9, "inter_node": 100e9 / 8, "latency": 20e-6,
            "hbm": 0.69e12, "bf16_flops": 1.2e14},
    "A10": {"mem_gb": 22.2, "intra_p2p": 22.8e9, "intra_allreduce_bus": 19.18e9, "inter_node": 40e9 / 8, "latency": 20e-6,
            "hbm": 0.6e12, "bf16_flops": 1.0e14},
}

# $ per hour for a node of `gpus_per_node` GPUs
PRICE_PER_NODE_HOUR = {"B200": 98.32, "A100": 32.7726, "A10": 8.144, "A40": 8.144}

# tokens per epoch-like unit used to turn step time into total time / cost (dataset -> number of sequences)
DATASETS = {"squad": 87599, "wikitext": 36718, "synthetic": 131072}


@dataclass
class ModelConfig:
    name: str
    num_layers: int
    hidden: int
    heads: int
    kv_heads: int
    ffn: int
    vocab: int
    seq_len: int
    head_dim: int = 0
    gated_mlp: bool = True

    def __post_init__(self):
        if not self.head_dim:
            self.head_dim = self.hidden // self.heads

    # ---- parameters per node (unsharded) -------------------------------------------------------
    def node_params(self, node: str) -> int:
        h, d = self.hidden, self.head_dim
        return {
            "embed": self.vocab * h,
            "attn_q": h + h * self.heads * d,            # input norm charged to q
            "attn_k": h * self.kv_heads * d,
            "attn_v": h * self.kv_heads * d,
            "attn_o": self.heads * d * h,
            "mlp_gate": h + h * self.ffn,                # post-attention norm charged to gate
            "mlp_act_fn": 0,
            "mlp_up": h * self.ffn if self.gated_mlp else 0,
            "mlp_down": self.ffn * h,
            "lm_head": h + h * self.vocab,
        }[node]

    def node_params_sharded(self, node: str, tp: int) -> float:
        p = self.node_params(node)
        if node in ("embed", "lm_head"):
            return p  # replicated in this framework
        norm = self.hidden if node in ("attn_q", "mlp_gate") else 0
        return (p - norm) / tp + norm

    def total_params(self) -> int:
        return sum(self.node_params(n) for n in ("embed", "lm_head")) + self.num_layers * sum(self.node_params(n) for n in LAYER_NODES)

    # ---- activation elements saved for backward per node, per token --------------------------------
    def node_act_elems(self, node: str, tp: int) -> float:
        h, d = self.hidden, self.head_dim
        return {
            "embed": h,
            "attn_q": h + self.heads * d / tp,           # norm input + q
            "attn_k": self.kv_heads * d / tp,
            "attn_v": self.kv_heads * d / tp,
            "attn_o": self.heads * d / tp + h,           # attention output + residual
            "mlp_gate": h + self.ffn / tp,
            "mlp_act_fn": self.ffn / tp,
            "mlp_up": self.ffn / tp,
            "mlp_down": h,
            "lm_head": h + self.vocab,
        }[node]

    # ---- elements crossing a pipeline cut placed AFTER this node, per token -------------------------------
    def cut_elems(self, node: str, tp: int, sequence_parallel: bool = True) -> float:
        return self.hidden / (tp if sequence_parallel else 1)

    def node_sequence(self) -> List[str]:
        return ["embed"] + list(LAYER_NODES) * self.num_layers + ["lm_head"]


MODEL_CONFIGS: Dict[str, ModelConfig] = {
    "llama1b": ModelConfig("llama1b", 16, 2048, 32, 8, 8192, 128256, 1024, head_dim=64),
    "llama3b": ModelConfig("llama3b", 28, 3072, 24, 8, 8192, 128256, 4096, head_dim=128),
    "llama8b": ModelConfig("llama8b", 32, 4096, 32, 8, 14336, 128256, 2048),
    "llama70b": ModelConfig("llama70b", 80, 8192, 64, 8, 28672, 128256, 1024),
    "gpt2XL": ModelConfig("gpt2XL", 48, 1600, 25, 25, 6400, 50257, 1024, gated_mlp=False),
    "bert": ModelConfig("bert", 24, 1024, 16, 16, 4096, 30522, 512, gated_mlp=False),
}
