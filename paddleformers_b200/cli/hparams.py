"""Argument dataclasses and the YAML / JSON / ``key=value`` parser of the command line.

Counterparts: paddleformers/cli/hparams/{model_args,data_args,finetuning_args,generating_args,export_args}.py and
``read_args`` / ``get_train_args`` (paddleformers/cli/hparams/parser.py:94, :212): one flat config file merged with
``key=value`` overrides, split over the dataclasses by field name; unknown keys are an error unless
``ALLOW_EXTRA_ARGS=1``.
"""
from __future__ import annotations

import dataclasses
import json
import os
import sys
import typing
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..trainer.training_args import TrainingArguments


@dataclass
class ModelArguments:
    model_name_or_path: Optional[str] = None
    model_type: Optional[str] = field(default=None, metadata={"help": "build from a named preset / model_type when no checkpoint is given"})
    stage: str = field(default="SFT", metadata={"help": "SFT | PT | DPO | VL-SFT | VL-PT | VL-DPO | auto-parallel | dsv3_pretrain | ernie_pretrain"})
    from_scratch: bool = False
    lora: bool = False
    lora_rank: int = 8
    lora_alpha: float = 16.0
    lora_dropout: float = 0.0
    rslora: bool = False
    lora_plus_scale: float = 1.0
    lora_target_modules: Optional[List[str]] = None
    lora_path: Optional[str] = None
    loraga: bool = False                 # initialise the adapters from full-weight gradients (LoRA-GA)
    loraga_init_iters: int = 8           # batches used for the gradient estimate
    loraga_stable_gamma: float = 16.0    # -1: scale the factors by 1 / lora scaling instead
    use_attn_mask_startend_row_indices: bool = True
    use_global_causal_attn: bool = False
    config_overrides: Optional[Dict[str, Any]] = None


@dataclass
class DataArguments:
    train_dataset_path: Optional[str] = None
    train_dataset_prob: Optional[str] = None
    eval_dataset_path: Optional[str] = None
    eval_dataset_prob: Optional[str] = None
    dataset_type: str = field(default="messages", metadata={"help": "messages | erniekit | pretrain (mmap)"})
    input_dir: Optional[str] = field(default=None, metadata={"help": "mmap dataset prefixes: 'w1 prefix1 w2 prefix2' or one prefix"})
    split: str = "949,50,1"
    template: Optional[str] = None
    packing: bool = True
    packing_strategy: str = "greedy"
    mix_strategy: str = "concat"
    padding_free: bool = False
    streaming: bool = False
    train_on_prompt: bool = False
    num_samples_each_epoch: int = 0
    min_pixels: Optional[int] = field(default=None, metadata={"help": "VL stages: lower bound of the resized image area"})
    max_pixels: Optional[int] = field(default=None, metadata={"help": "VL stages: upper bound of the resized image area"})


@dataclass
class GeneratingArguments:
    max_new_tokens: int = 64
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    num_beams: int = 1


@dataclass
class ExportArguments:
    export_dir: Optional[str] = None
    export_dtype: str = "bfloat16"


@dataclass
class FinetuningArguments(TrainingArguments):
    compute_type: str = field(default="bf16", metadata={"help": "bf16 | fp16 | float32 | wint8 | wint4 | nf4 | fp8"})
    dpo_beta: float = 0.1
    dpo_loss_type: str = "sigmoid"
    dpo_label_smoothing: float = 0.0
    sft_loss_ratio: float = 0.0
    ref_model_name_or_path: Optional[str] = None
    weight_quantize_algo: Optional[str] = None

    def __post_init__(self):
        ct = self.compute_type
        if ct in ("bf16", "bfloat16"):
            self.bf16 = True
        elif ct in ("fp16", "float16"):
            self.fp16 = True
        elif ct in ("wint8", "wint4", "nf4"):
            self.bf16, self.weight_quantize_algo = True, ct
        elif ct == "fp8":
            self.bf16, self.fp8 = True, "e4m3"
        elif ct not in ("float32", "fp32"):
            raise ValueError(f"unknown compute_type {ct!r}")
        super().__post_init__()


ARG_CLASSES = (ModelArguments, DataArguments, GeneratingArguments, ExportArguments, FinetuningArguments)


def _coerce(value, typ):
    if value is None or not isinstance(value, str):
        return value
    origin = typing.get_origin(typ)
    if origin is typing.Union:
        args = [a for a in typing.get_args(typ) if a is not type(None)]
        if value.lower() in ("none", "null"):
            return None
        return _coerce(value, args[0]) if args else value
    if typ is bool:
        return value.lower() in ("1", "true", "yes", "on")
    if typ is int:
        return int(value)
    if typ is float:
        return float(value)
    if origin in (list, List):
        return json.loads(value) if value.startswith("[") else [v for v in value.split(",") if v]
    if origin in (dict, Dict):
        return json.loads(value)
    return value


def read_args(argv: Optional[List[str]] = None) -> Dict[str, Any]:
    """``[config.yaml|config.json] [key=value ...]`` -> flat dict."""
    argv = list(sys.argv[1:] if argv is None else argv)
    cfg: Dict[str, Any] = {}
    if argv and (argv[0].endswith((".yaml", ".yml", ".json"))):
        path = argv.pop(0)
        with open(path) as f:
            if path.endswith(".json"):
                cfg = json.load(f)
            else:
                import yaml

                cfg = yaml.safe_load(f) or {}
    for item in argv:
        if "=" not in item:
            raise ValueError(f"override {item!r} is not of the form key=value")
        k, v = item.split("=", 1)
        cfg[k.lstrip("-")] = v
    return cfg


def parse_dict(cfg: Dict[str, Any], classes=ARG_CLASSES) -> Tuple:
    # keys that only the reference's trainer knows are translated, accepted without effect or refused with a pointer
    from .reference_flags import translate

    cfg = translate(cfg, {f.name for cls in classes for f in dataclasses.fields(cls)})
    used = set()
    outs = []
    hints_cache = {}
    for cls in classes:
        hints = typing.get_type_hints(cls)
        kwargs = {}
        for f in dataclasses.fields(cls):
            if f.name in cfg and f.init:
                kwargs[f.name] = _coerce(cfg[f.name], hints.get(f.name, str))
                used.add(f.name)
        outs.append(cls(**kwargs))
    extra = sorted(set(cfg) - used)
    if extra and os.environ.get("ALLOW_EXTRA_ARGS", "0") != "1":
        raise ValueError(f"unknown configuration keys: {extra} (set ALLOW_EXTRA_ARGS=1 to ignore)")
    return tuple(outs)


def get_train_args(argv: Optional[List[str]] = None):
    return parse_dict(read_args(argv))
