from .merge import MergeConfig, MergeModel, merge_lora_and_export  # noqa: F401
