"""Low-rank adapters (LoRA, DoRA, rsLoRA) and their PEFT folder format."""
from .lora import (DEFAULT_TARGETS, DoraAdapter, LoraAdapter, adapter_parameters, add_adapters, merge_adapters,
                   named_adapters, remove_adapters)

__all__ = ["DEFAULT_TARGETS", "DoraAdapter", "LoraAdapter", "adapter_parameters", "add_adapters", "merge_adapters",
           "named_adapters", "remove_adapters"]
