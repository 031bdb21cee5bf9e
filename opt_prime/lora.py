"""Compatibility alias of :mod:`aicomp_b200.lora` under the reference's module name."""
from aicomp_b200.lora import LoRAConfig, LoRALinear, LoRAAdapter, apply_lora_to_module, lora_state_dict, load_lora_state_dict  # noqa: F401
