from .lora import LoRAConfig, LoRALinear, LoRAModel, LoRAMoeExperts  # noqa: F401
