"""Model configuration base classes.

``PretrainedConfig`` reads / writes Hugging Face ``config.json`` files; ``LlmMetaConfig`` lists the run-time
attributes (fusion switches, parallel degrees, recompute, loss, MoE, MTP, fp8) that the trainer copies onto the model
config so that model code can read e.g. ``config.tensor_model_parallel_size`` or ``config.sequence_parallel``.
Same roles as paddleformers/transformers/configuration_utils.py:230-668 (LlmMetaConfig, set_llm_config) and :670
(PretrainedConfig) in the reference.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any, Dict, List, Optional, Tuple

CONFIG_NAME = "config.json"
GENERATION_CONFIG_NAME = "generation_config.json"


class LlmMetaConfig:
    """Declarative table of run-time attributes: (name, type, default, help)."""

    op_fusion_attributes = [
        ("use_fused_linear_cross_entropy", bool, False, "fuse lm_head GEMM with the cross entropy"),
        ("apply_rope_fusion", bool, True, "use the fused RoPE kernel"),
        ("fuse_swiglu", bool, True, "run SwiGLU in the gate/up GEMM epilogue"),
        ("fuse_attention_qkv", bool, True, "single fused qkv projection"),
        ("fuse_attention_ffn", bool, True, "single fused gate/up projection"),
        ("fuse_rms_norm", bool, True, "use the fused RMSNorm(+residual) kernel"),
    ]
    hybrid_parallel_attributes = [
        ("tensor_model_parallel_size", int, 1, "tensor parallel degree"),
        ("tensor_parallel_rank", int, 0, "rank inside the tensor parallel group"),
        ("tensor_parallel_output", bool, True, "keep lm_head logits vocabulary-sharded"),
        ("pipeline_model_parallel_size", int, 1, "pipeline parallel degree"),
        ("virtual_pipeline_model_parallel_size", int, 1, "interleaved pipeline chunks per stage"),
        ("pipeline_schedule", str, "1F1B", "1F1B | interleaved | FThenB | zero_bubble | zbv (V-shaped placement, two chunks per stage)"),
        ("num_empty_layers_add_in_head", int, 0, "empty layers inserted before the first decoder layer"),
        ("num_empty_layers_add_in_tail", int, 0, "empty layers appended after the last decoder layer"),
        ("expert_model_parallel_size", int, 1, "expert parallel degree"),
        ("context_parallel_size", int, 1, "context parallel degree"),
        ("cp_balance_mode", str, "dualchunk_allgather", "dualchunk_allgather (zig-zag) or contiguous_allgather"),
        ("context_parallel_algo", str, "allgather", "allgather (gather K/V over the cp group) | ring (K/V ring with log-sum-exp merging)"),
        ("sep_parallel_size", int, 1, "Ulysses (segment) parallel degree"),
        ("sequence_parallel", bool, False, "Megatron sequence parallel inside the tensor parallel group"),
        ("fuse_sequence_parallel_allreduce", bool, False, "fuse SP parameter gradient all-reduces"),
        ("no_recompute_layers", Optional[List[int]], None, "layers excluded from recompute"),
    ]
    recompute_attributes = [
        ("recompute_granularity", Optional[str], None, "full | selective | None"),
        ("recompute_method", Optional[str], None, "uniform | block"),
        ("recompute_num_layers", int, 1, "layers per recompute chunk"),
        ("recompute_modules", Optional[Any], None, "module names to recompute under selective granularity"),
        ("recompute_use_reentrant", bool, False, "use the reentrant checkpoint implementation"),
        ("refined_recompute", Optional[Any], None, "with full recompute: {operation: number of layers that recompute it} for "
         "attention_column_ln | flash_attn | attention_row_ln | mlp_column_ln | mlp_row_ln; the other layers keep that "
         "operation's saved tensors (0: kept in every layer)"),
    ]
    loss_attributes = [
        ("use_fused_head_and_loss_fn", bool, False, "fused head + loss computing gradients in the forward"),
        ("use_filtered_label_loss", bool, False, "compute logits only at non-ignored label positions"),
        ("loss_subbatch_sequence_length", int, -1, "chunk length of the head/loss computation"),
    ]
    moe_attributes = [
        ("moe_router_force_load_balancing", bool, False, "route tokens round-robin (benchmarking aid)"),
        ("moe_router_load_balancing_type", str, "aux_loss", "aux_loss | seq_aux_loss | none"),
        ("moe_token_dispatcher_type", str, "fused", "fused (NVSwitch kernel) | alltoall (NCCL baseline)"),
        ("moe_grouped_gemm", bool, True, "use the grouped expert GEMM"),
        ("moe_subbatch_token_num_before_dispatch", int, 0, "split tokens into sub-batches before dispatch"),
    ]
    mtp_attributes = [
        ("train_mtp_only", int, 0, "train MTP layers only"),
        ("num_nextn_predict_layers", int, 0, "number of multi-token-prediction layers"),
        ("mtp_loss_scaling_factor", float, 0.1, "weight of the averaged MTP losses"),
    ]
    fp8_attributes = [
        ("fp8", Optional[str], None, "None | e4m3 block-scaled training"),
        ("use_ue8m0", bool, True, "power-of-two (UE8M0) block scales"),
    ]
    model_attributes = [
        ("fa_version", int, 4, "attention kernel generation (kept for CLI compatibility)"),
        ("_attn_implementation", str, "flashmask", "eager | sdpa | flashmask"),
    ]

    @classmethod
    def _get_all_meta(cls) -> List[Tuple[str, Any, Any, str]]:
        out = []
        for name in dir(cls):
            if name.endswith("_attributes"):
                out.extend(getattr(cls, name))
        return out

    @classmethod
    def _get_defaults(cls) -> Dict[str, Any]:
        return {n: copy.deepcopy(d) for n, _, d, _ in cls._get_all_meta()}

    @classmethod
    def _get_unsavable_keys(cls) -> List[str]:
        return [n for n, _, _, _ in cls._get_all_meta()]

    @classmethod
    def set_llm_config(cls, config, args) -> None:
        """Copy every meta attribute that ``args`` defines onto ``config``."""
        for name, _, _, _ in cls._get_all_meta():
            if hasattr(args, name):
                val = getattr(args, name)
                if val is not None:
                    setattr(config, name, val)


def llmmetaclass(cls):
    """Class decorator that injects every LlmMetaConfig attribute as a dataclass field (used by the argument
    dataclasses so that each model-side switch is also a CLI flag)."""
    import dataclasses

    ann = dict(getattr(cls, "__annotations__", {}))
    for name, typ, default, help_ in LlmMetaConfig._get_all_meta():
        if name in ann or name.startswith("_"):
            continue
        ann[name] = Optional[typ] if typ in (bool, int, float, str) else typ
        setattr(cls, name, dataclasses.field(default=None, metadata={"help": help_}))
    cls.__annotations__ = ann
    return cls


class PretrainedConfig:
    model_type: str = ""
    # fields whose null is a value of its own and differs from other loaders' defaults (no low-rank query projection, no window)
    keep_null_keys = ("q_lora_rank", "sliding_window")
    attribute_map: Dict[str, str] = {}

    def __init__(self, **kwargs):
        for k, v in LlmMetaConfig._get_defaults().items():
            setattr(self, k, kwargs.pop(k, v))
        self.vocab_size = kwargs.pop("vocab_size", 32000)
        self.hidden_size = kwargs.pop("hidden_size", 4096)
        self.num_hidden_layers = kwargs.pop("num_hidden_layers", 32)
        self.num_attention_heads = kwargs.pop("num_attention_heads", 32)
        self.tie_word_embeddings = kwargs.pop("tie_word_embeddings", False)
        self.initializer_range = kwargs.pop("initializer_range", 0.02)
        self.dtype = kwargs.pop("dtype", kwargs.pop("torch_dtype", "float32"))
        self.bos_token_id = kwargs.pop("bos_token_id", None)
        self.eos_token_id = kwargs.pop("eos_token_id", None)
        self.pad_token_id = kwargs.pop("pad_token_id", None)
        self.architectures = kwargs.pop("architectures", None)
        self.use_cache = kwargs.pop("use_cache", True)
        self.quantization_config = kwargs.pop("quantization_config", None)
        kwargs.pop("model_type", None)
        kwargs.pop("transformers_version", None)
        for k, v in kwargs.items():
            setattr(self, k, v)

    def __getattr__(self, name):
        amap = type(self).attribute_map
        if name in amap:
            return getattr(self, amap[name])
        raise AttributeError(f"{type(self).__name__} has no attribute {name!r}")

    # ------------------------------------------------------------------ serialisation
    def to_dict(self, saving: bool = False) -> Dict[str, Any]:
        out = {}
        skip = set(LlmMetaConfig._get_unsavable_keys()) if saving else set()
        for k, v in self.__dict__.items():
            if k in skip or k.startswith("_"):
                continue
            if hasattr(v, "to_dict"):
                v = v.to_dict()
            if saving and v is None and k not in self.keep_null_keys:
                continue          # absent == None on load; an explicit null breaks other loaders (quantization_config)
            out[k] = v
        out["model_type"] = self.model_type
        if saving:
            out["torch_dtype"] = out.get("dtype", "float32")
        return out

    def to_json_string(self, saving: bool = False) -> str:
        return json.dumps(self.to_dict(saving), indent=2, sort_keys=True, default=str) + "\n"

    def save_pretrained(self, save_directory: str) -> None:
        os.makedirs(save_directory, exist_ok=True)
        with open(os.path.join(save_directory, CONFIG_NAME), "w") as f:
            f.write(self.to_json_string(saving=True))

    @classmethod
    def from_dict(cls, d: Dict[str, Any], **overrides) -> "PretrainedConfig":
        d = dict(d)
        d.update(overrides)
        return cls(**d)

    @classmethod
    def get_config_dict(cls, path: str) -> Dict[str, Any]:
        from ..utils.download import resolve_file_path

        file = path if os.path.isfile(path) else resolve_file_path(path, CONFIG_NAME)
        with open(file) as f:
            return json.load(f)

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "PretrainedConfig":
        return cls.from_dict(cls.get_config_dict(path), **overrides)

    def __repr__(self):
        return f"{type(self).__name__} {self.to_json_string()}"

    # convenience used by model code
    @property
    def head_dim_(self) -> int:
        hd = self.__dict__.get("head_dim", None)
        return hd if hd else self.hidden_size // self.num_attention_heads
