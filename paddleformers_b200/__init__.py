"""B200-native LLM training framework with the capabilities of PaddleFormers.

Public entry points (lazily imported so that ``import paddleformers_b200`` stays cheap, like the reference's
``_LazyModule`` shim, paddleformers/utils/lazy_import.py):

    AutoConfig, AutoModelForCausalLM, AutoTokenizer        model API
    Trainer, TrainingArguments                             training API
    paddleformers_b200.ops.functional                      sm_100a kernels behind torch autograd
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_LAZY = {
    "AutoConfig": ".transformers.auto", "AutoModelForCausalLM": ".transformers.auto", "AutoTokenizer": ".transformers.auto",
    "AutoModelForCausalLMPipe": ".transformers.auto", "AutoProcessor": ".transformers.auto",
    "PretrainedConfig": ".transformers.configuration_utils", "PretrainedModel": ".transformers.model_utils",
    "Trainer": ".trainer.trainer", "TrainingArguments": ".trainer.training_args",
    "TrainerCallback": ".trainer.trainer_callback",
    "LlamaForCausalLM": ".models.modeling", "Qwen3ForCausalLM": ".models.modeling", "Qwen3MoeForCausalLM": ".models.modeling",
    "DeepseekV3ForCausalLM": ".models.modeling", "Glm4MoeForCausalLM": ".models.modeling",
    "LlamaConfig": ".models.configuration", "Qwen3Config": ".models.configuration", "Qwen3MoeConfig": ".models.configuration",
    "DeepseekV3Config": ".models.configuration", "Glm4MoeConfig": ".models.configuration",
    "LoRAConfig": ".peft.lora", "LoRAModel": ".peft.lora", "GenerationConfig": ".generation.utils",
    "AutoModelForConditionalGeneration": ".transformers.auto", "Qwen2VLForConditionalGeneration": ".models.vision_language",
    "Qwen2VLConfig": ".models.vision_language", "Qwen2_5_VLConfig": ".models.vision_language",
    "Qwen2_5_VLForConditionalGeneration": ".models.vision_language", "Qwen2VLImageProcessor": ".transformers.image_processing",
    "Qwen2ForCausalLM": ".models.modeling", "MistralForCausalLM": ".models.modeling", "Phi3ForCausalLM": ".models.modeling",
    "Ernie4_5ForCausalLM": ".models.modeling", "Ernie4_5MoeForCausalLM": ".models.modeling", "Qwen2MoeForCausalLM": ".models.modeling",
    "GraniteForCausalLM": ".models.modeling", "SFTTrainer": ".trainer.sft_trainer", "DPOTrainer": ".trainer.dpo_trainer",
    "ShardedAdamW": ".parallel.sharding", "ShardedMuon": ".parallel.sharding", "EMACallback": ".trainer.ema",
    "plan_parallelism": ".parallel.auto_plan",
    "PaliGemmaForConditionalGeneration": ".models.paligemma", "Gemma3ForConditionalGeneration": ".models.paligemma",
    "AutoModelForSpeechSeq2Seq": ".transformers.auto", "WhisperForConditionalGeneration": ".models.whisper",
    "AutoModelForSequenceClassification": ".transformers.auto", "AutoModelForTokenClassification": ".transformers.auto",
    "AutoModel": ".transformers.auto", "SiglipVisionModel": ".models.siglip", "SiglipVisionConfig": ".models.siglip",
    "Qwen3VLForConditionalGeneration": ".models.vision_language", "Qwen3VLMoeForConditionalGeneration": ".models.vision_language",
    "Glm4vMoeForConditionalGeneration": ".models.vision_language", "FullyShardedOptimizer": ".parallel.fsdp",
    "Gemma4ForCausalLM": ".models.gemma4", "Gemma4TextConfig": ".models.gemma4",
    "MolmoForCausalLM": ".models.molmo", "MolmoConfig": ".models.molmo",
    "Phi4MultimodalForCausalLM": ".models.phi4_multimodal", "Phi4MultimodalConfig": ".models.phi4_multimodal",
    "Ernie4_5VLForConditionalGeneration": ".models.ernie4_5_vl", "Ernie4_5VLConfig": ".models.ernie4_5_vl",
}


def __getattr__(name):
    if name in _LAZY:
        mod = importlib.import_module(_LAZY[name], __name__)
        return getattr(mod, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
