"""Auto classes: pick the config / model / tokenizer class from ``model_type`` in ``config.json``.

Same entry points as the reference (paddleformers/transformers/auto/modeling.py:774 AutoModelForCausalLM, AutoConfig,
AutoTokenizer). Tokenizers are thin wrappers over Hugging Face ``transformers`` tokenizers, like the reference's
(paddleformers/transformers/llama/tokenizer.py:21-22).
"""
from __future__ import annotations

from typing import Optional

from .configuration_utils import PretrainedConfig


class AutoConfig:
    @staticmethod
    def for_model(model_type: str, **kw) -> PretrainedConfig:
        from ..models.configuration import resolve_config_class

        return resolve_config_class(model_type)(**kw)

    @staticmethod
    def from_pretrained(path: str, **overrides) -> PretrainedConfig:
        from ..models.configuration import resolve_config_class

        d = PretrainedConfig.get_config_dict(path)
        return resolve_config_class(d.get("model_type")).from_dict(d, **overrides)


class AutoModelForCausalLM:
    @staticmethod
    def _cls(config):
        from ..models.modeling import MODEL_MAPPING

        return MODEL_MAPPING[config.model_type]

    @classmethod
    def from_config(cls, config: PretrainedConfig, dtype=None, device=None, **kw):
        return cls._cls(config).from_config(config, dtype=dtype, device=device, **kw)

    @classmethod
    def from_pretrained(cls, path: str, config: Optional[PretrainedConfig] = None, dtype=None, device=None, **kw):
        config = config or AutoConfig.from_pretrained(path)
        return cls._cls(config).from_pretrained(path, config=config, dtype=dtype, device=device, **kw)


class AutoModelForConditionalGeneration:
    """Vision-language models (image / video placeholders in the token stream)."""

    @staticmethod
    def _classes(model_type: str):
        from ..models.vision_language import (Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration, Qwen2VLConfig,
                                              Qwen2VLForConditionalGeneration, Qwen3VLConfig, Qwen3VLForConditionalGeneration,
                                              Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration, Glm4vMoeConfig,
                                              Glm4vMoeForConditionalGeneration, GlmOcrConfig, GlmOcrForConditionalGeneration)
        from ..models.paligemma import (AyaVisionConfig, AyaVisionForConditionalGeneration, Gemma3Config,
                                        Gemma3ForConditionalGeneration, PaliGemma2Config, PaliGemmaConfig,
                                        PaliGemmaForConditionalGeneration, ShieldGemma2Config, ShieldGemma2ForImageClassification)

        from ..models.llama4_vision import Llama4Config, Llama4ForConditionalGeneration

        from ..models.paddleocr_vl import PaddleOCRVLConfig, PaddleOCRVLForConditionalGeneration

        from ..models.ernie4_5_vl import Ernie4_5VLConfig, Ernie4_5VLForConditionalGeneration

        from ..models.phi4_multimodal import Phi4MultimodalConfig, Phi4MultimodalForCausalLM

        from ..models.molmo import MolmoConfig, MolmoForCausalLM

        table = {"molmo": (MolmoConfig, MolmoForCausalLM),
                 "phi4_multimodal": (Phi4MultimodalConfig, Phi4MultimodalForCausalLM),
                 "phi4mm": (Phi4MultimodalConfig, Phi4MultimodalForCausalLM),
                 "ernie4_5_vl_moe": (Ernie4_5VLConfig, Ernie4_5VLForConditionalGeneration),
                 "ernie4_5_moe_vl": (Ernie4_5VLConfig, Ernie4_5VLForConditionalGeneration),      # the reference's spelling
                 "llama4": (Llama4Config, Llama4ForConditionalGeneration),
                 "paddleocr_vl": (PaddleOCRVLConfig, PaddleOCRVLForConditionalGeneration),
                 "paligemma": (PaliGemmaConfig, PaliGemmaForConditionalGeneration),
                 "paligemma2": (PaliGemma2Config, PaliGemmaForConditionalGeneration),
                 "gemma3": (Gemma3Config, Gemma3ForConditionalGeneration),
                 "aya_vision": (AyaVisionConfig, AyaVisionForConditionalGeneration),
                 "shieldgemma2": (ShieldGemma2Config, ShieldGemma2ForImageClassification),
                 "qwen2_vl": (Qwen2VLConfig, Qwen2VLForConditionalGeneration),
                 "qwen2_5_vl": (Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration),
                 "qwen3_vl": (Qwen3VLConfig, Qwen3VLForConditionalGeneration),
                 "qwen3_vl_moe": (Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration),
                 "glm4v_moe": (Glm4vMoeConfig, Glm4vMoeForConditionalGeneration),
                 "glm_ocr": (GlmOcrConfig, GlmOcrForConditionalGeneration)}
        if model_type not in table:
            raise ValueError(f"unknown vision-language model_type {model_type!r}; supported: {sorted(table)}")
        return table[model_type]

    @classmethod
    def from_config(cls, config, dtype=None, device=None, **kw):
        return cls._classes(config.model_type)[1].from_config(config, dtype=dtype, device=device, **kw)

    @classmethod
    def from_pretrained(cls, path: str, dtype=None, device=None, **kw):
        mt = PretrainedConfig.get_config_dict(path).get("model_type")
        cfg_cls, model_cls = cls._classes(mt)
        return model_cls.from_pretrained(path, config=cfg_cls.from_pretrained(path), dtype=dtype, device=device, **kw)


class AutoModel:
    """Encoders without a language-model head (image towers)."""

    @staticmethod
    def _classes(model_type: str):
        from ..models.siglip import SiglipVisionConfig, SiglipVisionModel

        table = {"siglip_vision_model": (SiglipVisionConfig, SiglipVisionModel)}
        if model_type not in table:
            raise ValueError(f"unknown encoder model_type {model_type!r}; supported: {sorted(table)}")
        return table[model_type]

    @classmethod
    def from_config(cls, config, dtype=None, device=None, **kw):
        return cls._classes(config.model_type)[1].from_config(config, dtype=dtype, device=device, **kw)

    @classmethod
    def from_pretrained(cls, path: str, dtype=None, device=None, **kw):
        mt = PretrainedConfig.get_config_dict(path).get("model_type")
        cfg_cls, model_cls = cls._classes(mt)
        return model_cls.from_pretrained(path, config=cfg_cls.from_pretrained(path), dtype=dtype, device=device, **kw)


class AutoModelForSequenceClassification:
    """Any supported decoder family with one label (or score) per sequence."""

    _kind = "DecoderForSequenceClassification"

    @classmethod
    def _cls(cls):
        from ..models import classification

        return getattr(classification, cls._kind)

    @classmethod
    def from_config(cls, config, dtype=None, device=None, **kw):
        return cls._cls().from_config(config, dtype=dtype, device=device, **kw)

    @classmethod
    def from_pretrained(cls, path: str, config=None, dtype=None, device=None, num_labels: Optional[int] = None, **kw):
        config = config or AutoConfig.from_pretrained(path)
        if num_labels is not None:
            config.num_labels = int(num_labels)
        return cls._cls().from_pretrained(path, config=config, dtype=dtype, device=device, **kw)


class AutoModelForTokenClassification(AutoModelForSequenceClassification):
    _kind = "DecoderForTokenClassification"


class AutoModelForSpeechSeq2Seq(AutoModel):
    """Encoder-decoder speech models."""

    @staticmethod
    def _classes(model_type: str):
        from ..models.whisper import WhisperConfig, WhisperForConditionalGeneration

        table = {"whisper": (WhisperConfig, WhisperForConditionalGeneration)}
        if model_type not in table:
            raise ValueError(f"unknown speech model_type {model_type!r}; supported: {sorted(table)}")
        return table[model_type]


class AutoModelForCausalLMPipe(AutoModelForCausalLM):
    """Pipeline-parallel variant: builds only this stage's layers (see ``parallel.pipeline``)."""

    @classmethod
    def from_config(cls, config: PretrainedConfig, dtype=None, device=None, **kw):
        from ..parallel.pipeline import build_pipeline_model

        return build_pipeline_model(config, dtype=dtype, device=device, **kw)

    @classmethod
    def from_pretrained(cls, path: str, config: Optional[PretrainedConfig] = None, dtype=None, device=None, **kw):
        from ..parallel.pipeline import PipelineStageModel

        config = config or AutoConfig.from_pretrained(path)
        return PipelineStageModel.from_pretrained(path, config=config, dtype=dtype, device=device, **kw)


class AutoTokenizer:
    @staticmethod
    def from_pretrained(path: str, **kw):
        from ..utils.download import resolve_dir

        try:
            from transformers import AutoTokenizer as HFAutoTokenizer
        except Exception as e:  # pragma: no cover
            raise RuntimeError("AutoTokenizer needs the `transformers` package") from e
        try:
            path = resolve_dir(path)
        except FileNotFoundError:
            pass
        return HFAutoTokenizer.from_pretrained(path, **kw)


class AutoProcessor:
    """Processors of this package for the directories that name them (Kimi-K2.5: ``KimiK25VisionProcessor`` in
    ``preprocessor_config.json``); every other directory goes to the `transformers` package."""

    @staticmethod
    def from_pretrained(path: str, **kw):
        import json
        import os

        pre = os.path.join(path, "preprocessor_config.json")
        if os.path.isfile(pre):
            with open(pre) as f:
                kind = json.load(f).get("image_processor_type")
            if kind == "KimiK25VisionProcessor":
                from .kimi_processing import KimiProcessor

                return KimiProcessor.from_pretrained(path)
        from transformers import AutoProcessor as HFAutoProcessor

        return HFAutoProcessor.from_pretrained(path, **kw)
