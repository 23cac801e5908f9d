"""Configurations of the supported decoder families (Hugging Face field names, so ``config.json`` files load as is).

Reference counterparts: paddleformers/transformers/llama/configuration.py, qwen2, qwen3,
qwen3_moe/configuration.py:154-226, deepseek_v3/configuration.py:136-238, glm4_moe/configuration.py:128-220.
"""
from __future__ import annotations

from typing import List, Optional

from ..transformers.configuration_utils import PretrainedConfig


class DecoderConfig(PretrainedConfig):
    """Superset of the per-family options read by the unified decoder implementation."""

    model_type = "decoder"

    def __init__(self, vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=None, head_dim=None, hidden_act="silu",
                 max_position_embeddings=4096, rms_norm_eps=1e-6, rope_theta=10000.0, rope_scaling=None, rope_parameters=None,
                 partial_rotary_factor=1.0, attention_bias=False, mlp_bias=False, use_qk_norm=False,
                 attention_dropout=0.0,
                 # MoE
                 num_experts=0, n_routed_experts=None, num_local_experts=None, num_experts_per_tok=0, moe_intermediate_size=None,
                 n_shared_experts=0, shared_expert_intermediate_size=None, first_k_dense_replace=0,
                 decoder_sparse_step=1, mlp_only_layers=None, norm_topk_prob=True, scoring_func="softmax",
                 topk_method="greedy", n_group=1, topk_group=1, routed_scaling_factor=1.0,
                 router_aux_loss_coef=0.0, router_z_loss_coef=0.0, output_router_logits=False,
                 # MLA
                 q_lora_rank=None, kv_lora_rank=None, qk_nope_head_dim=None, qk_rope_head_dim=None, v_head_dim=None,
                 **kwargs):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, num_hidden_layers=num_hidden_layers,
                         num_attention_heads=num_attention_heads, **kwargs)
        self.intermediate_size = intermediate_size
        self.num_key_value_heads = num_key_value_heads or num_attention_heads
        self.head_dim = head_dim or hidden_size // num_attention_heads
        self.hidden_act = hidden_act
        self.max_position_embeddings = max_position_embeddings
        self.rms_norm_eps = rms_norm_eps
        if rope_parameters:          # recent Hugging Face configs: base and scaling rule in one dict
            rope_theta = rope_parameters.get("rope_theta", rope_theta)
            kind = rope_parameters.get("rope_type", rope_parameters.get("type", "default"))
            if kind not in (None, "default") and rope_scaling is None:
                rope_scaling = {k: v for k, v in rope_parameters.items() if k != "rope_theta"}
            if "partial_rotary_factor" in rope_parameters and partial_rotary_factor == 1.0:
                partial_rotary_factor = rope_parameters["partial_rotary_factor"]
        self.rope_theta = rope_theta
        self.rope_scaling = rope_scaling
        self.partial_rotary_factor = partial_rotary_factor
        self.attention_bias = attention_bias
        self.mlp_bias = mlp_bias
        self.use_qk_norm = use_qk_norm
        self.attention_dropout = attention_dropout
        if num_local_experts is not None and not num_experts:      # the name recent Hugging Face configs serialise
            num_experts = num_local_experts
        self.num_experts = n_routed_experts if n_routed_experts is not None else num_experts
        self.num_experts_per_tok = num_experts_per_tok
        self.moe_intermediate_size = moe_intermediate_size
        self.n_shared_experts = n_shared_experts or 0
        self.shared_expert_intermediate_size = shared_expert_intermediate_size
        self.first_k_dense_replace = first_k_dense_replace
        self.decoder_sparse_step = decoder_sparse_step
        self.mlp_only_layers = mlp_only_layers or []
        self.norm_topk_prob = norm_topk_prob
        self.scoring_func = scoring_func
        self.topk_method = topk_method
        self.n_group = n_group
        self.topk_group = topk_group
        self.routed_scaling_factor = routed_scaling_factor
        self.router_aux_loss_coef = router_aux_loss_coef
        self.router_z_loss_coef = router_z_loss_coef
        self.output_router_logits = output_router_logits
        self.q_lora_rank = q_lora_rank
        self.kv_lora_rank = kv_lora_rank
        self.qk_nope_head_dim = qk_nope_head_dim
        self.qk_rope_head_dim = qk_rope_head_dim
        self.v_head_dim = v_head_dim

    @property
    def n_routed_experts(self):
        return self.num_experts

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if self.num_experts and self.model_type in ("deepseek_v3", "deepseek_v2", "deepseek_v32", "glm4_moe", "glm4_moe_lite", "glm_moe_dsa", "kimi_k2"):
            d["n_routed_experts"] = self.num_experts      # the field name these families use in config.json
            d.pop("num_experts", None)
        return d

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank is not None

    def layer_window(self, layer_idx: int) -> int:
        """Sliding-window width of a layer (0 = full causal attention): query i sees keys j with i - j < window. All layers
        use ``sliding_window`` unless ``layer_types`` names the kind of each layer ("sliding_attention" / "full_attention")
        or, Qwen2 style, ``use_sliding_window`` with ``max_window_layers`` (layers from that index on slide)."""
        w = int(getattr(self, "sliding_window", 0) or 0)
        if w <= 0:
            return 0
        types = getattr(self, "layer_types", None)
        if types:
            return w if (layer_idx < len(types) and types[layer_idx] == "sliding_attention") else 0
        if getattr(self, "use_sliding_window", None) is not None:
            return w if (self.use_sliding_window and layer_idx >= int(getattr(self, "max_window_layers", 0) or 0)) else 0
        return w

    def layer_chunk(self, layer_idx: int) -> int:
        """Chunk length of a chunked-attention layer (0 = none): a query sees the keys of its own chunk of ``attention_chunk_size``
        consecutive positions only (Llama 4's local layers)."""
        c = int(getattr(self, "attention_chunk_size", 0) or 0)
        types = getattr(self, "layer_types", None)
        if c <= 0 or not types or layer_idx >= len(types):
            return 0
        return c if types[layer_idx] == "chunked_attention" else 0

    def is_moe_layer(self, layer_idx: int) -> bool:
        if getattr(self, "moe_layers", None) is not None and self.num_experts > 0:
            return layer_idx in self.moe_layers
        if self.num_experts <= 0:
            return False
        if layer_idx in self.mlp_only_layers or layer_idx < self.first_k_dense_replace:
            return False
        return (layer_idx + 1) % max(self.decoder_sparse_step, 1) == 0


class LlamaConfig(DecoderConfig):
    model_type = "llama"

    def __init__(self, **kw):
        kw.setdefault("rms_norm_eps", 1e-6)
        super().__init__(**kw)
        self.attention_out_bias = bool(self.attention_bias)      # Llama's switch covers the output projection too


class Qwen2Config(DecoderConfig):
    model_type = "qwen2"

    def __init__(self, **kw):
        kw.setdefault("attention_bias", True)
        super().__init__(**kw)


class Qwen3Config(DecoderConfig):
    model_type = "qwen3"

    def __init__(self, **kw):
        kw.setdefault("use_qk_norm", True)
        kw.setdefault("head_dim", 128)
        super().__init__(**kw)


def _expert_count_alias(kw):
    """Recent Hugging Face releases serialise the expert count of these families as ``num_local_experts``."""
    if "num_local_experts" in kw and "num_experts" not in kw:
        kw["num_experts"] = kw["num_local_experts"]


class Qwen3MoeConfig(DecoderConfig):
    model_type = "qwen3_moe"

    def __init__(self, **kw):
        _expert_count_alias(kw)
        kw.setdefault("use_qk_norm", True)
        kw.setdefault("head_dim", 128)
        kw.setdefault("num_experts", 128)
        kw.setdefault("num_experts_per_tok", 8)
        kw.setdefault("moe_intermediate_size", 768)
        kw.setdefault("norm_topk_prob", True)
        kw.setdefault("router_aux_loss_coef", 1e-3)
        kw.setdefault("scoring_func", "softmax")
        super().__init__(**kw)


class DeepseekV3Config(DecoderConfig):
    model_type = "deepseek_v3"

    def __init__(self, **kw):
        kw.setdefault("hidden_size", 7168)
        kw.setdefault("intermediate_size", 18432)
        kw.setdefault("moe_intermediate_size", 2048)
        kw.setdefault("num_attention_heads", 128)
        kw.setdefault("num_key_value_heads", 128)
        if "num_experts" not in kw:
            kw.setdefault("n_routed_experts", 256)
        kw.setdefault("n_shared_experts", 1)
        kw.setdefault("num_experts_per_tok", 8)
        kw.setdefault("first_k_dense_replace", 3)
        kw.setdefault("scoring_func", "sigmoid")
        kw.setdefault("topk_method", "noaux_tc")
        kw.setdefault("n_group", 8)
        kw.setdefault("topk_group", 4)
        kw.setdefault("routed_scaling_factor", 2.5)
        kw.setdefault("q_lora_rank", 1536)
        kw.setdefault("kv_lora_rank", 512)
        kw.setdefault("qk_nope_head_dim", 128)
        kw.setdefault("qk_rope_head_dim", 64)
        kw.setdefault("v_head_dim", 128)
        kw.setdefault("head_dim", 192)
        kw.setdefault("vocab_size", 129280)
        kw.setdefault("num_nextn_predict_layers", 1)
        super().__init__(**kw)


class Glm4MoeLiteConfig(DeepseekV3Config):
    """GLM-4.7-Flash class models (``glm4_moe_lite``): DeepSeek-V3's blocks (multi-head latent attention with interleaved rotary
    rows, sigmoid ``noaux_tc`` routing, shared expert) at other sizes, without a multi-token-prediction layer; ``mlp_layer_types``
    lists which layers are dense."""

    model_type = "glm4_moe_lite"

    def __init__(self, mlp_layer_types=None, **kw):
        kw.setdefault("hidden_size", 2048)
        kw.setdefault("intermediate_size", 10240)
        kw.setdefault("moe_intermediate_size", 1536)
        kw.setdefault("num_attention_heads", 20)
        kw.setdefault("num_key_value_heads", kw["num_attention_heads"])
        if "num_experts" not in kw:
            kw.setdefault("n_routed_experts", 64)
        kw.setdefault("num_experts_per_tok", 4)
        kw.setdefault("n_group", 1)
        kw.setdefault("topk_group", 1)
        kw.setdefault("routed_scaling_factor", 1.8)
        kw.setdefault("q_lora_rank", 768)
        kw.setdefault("kv_lora_rank", 512)
        kw.setdefault("qk_nope_head_dim", 192)
        kw.setdefault("qk_rope_head_dim", 64)
        kw.setdefault("v_head_dim", 256)
        kw["head_dim"] = kw["qk_nope_head_dim"] + kw["qk_rope_head_dim"]
        kw.setdefault("rms_norm_eps", 1e-5)
        kw.setdefault("vocab_size", 154880)
        kw.setdefault("num_nextn_predict_layers", 0)
        if mlp_layer_types:
            dense = [i for i, t in enumerate(mlp_layer_types) if t == "dense"]
            if dense != list(range(len(dense))):
                raise NotImplementedError("dense layers are expected at the start of the stack")
            kw["first_k_dense_replace"] = len(dense)
        else:
            kw.setdefault("first_k_dense_replace", 1)
        super().__init__(**kw)

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            d["mlp_layer_types"] = ["dense" if i < self.first_k_dense_replace else "sparse" for i in range(self.num_hidden_layers)]
            d["qk_head_dim"] = self.qk_nope_head_dim + self.qk_rope_head_dim
            d.pop("head_dim", None)          # other loaders read it as the rotary width of the latent attention
        return d


class GlmMoeDsaConfig(Glm4MoeLiteConfig):
    """GLM with DeepSeek sparse attention (``glm_moe_dsa``): latent attention whose queries attend to the ``index_topk`` keys
    picked by a light indexer (``index_n_heads`` x ``index_head_dim``); sequences no longer than ``index_topk`` are plain
    latent attention."""

    model_type = "glm_moe_dsa"

    def __init__(self, index_topk=2048, index_n_heads=32, index_head_dim=128, **kw):
        kw.setdefault("routed_scaling_factor", 2.5)
        super().__init__(**kw)
        self.index_topk, self.index_n_heads, self.index_head_dim = index_topk, index_n_heads, index_head_dim
        self.no_kv_cache = True
        self.rope_interleave = False          # checkpoints of this family store half-split rotary rows


class DeepseekV32Config(DeepseekV3Config):
    """DeepSeek-V3.2: DeepSeek-V3 with the sparse-attention indexer (paddleformers/transformers/deepseek_v32)."""

    model_type = "deepseek_v32"

    def __init__(self, index_topk=2048, index_n_heads=64, index_head_dim=128, **kw):
        super().__init__(**kw)
        self.index_topk, self.index_n_heads, self.index_head_dim = index_topk, index_n_heads, index_head_dim
        self.no_kv_cache = True


class DeepseekV2Config(DeepseekV3Config):
    """DeepSeek-V2 / V2-Lite: MLA with a softmax router (greedy or group-limited), no multi-token-prediction layer, the query
    projected directly when ``q_lora_rank`` is null (paddleformers/transformers/deepseek_v3 serves both generations)."""

    model_type = "deepseek_v2"

    def __init__(self, **kw):
        kw.setdefault("scoring_func", "softmax")
        kw.setdefault("topk_method", "greedy")
        kw.setdefault("norm_topk_prob", False)
        kw.setdefault("routed_scaling_factor", 1.0)
        kw.setdefault("num_nextn_predict_layers", 0)
        kw.setdefault("first_k_dense_replace", 1)
        if "num_experts" not in kw:
            kw.setdefault("n_routed_experts", 64)
        kw.setdefault("num_experts_per_tok", 6)
        kw.setdefault("n_shared_experts", 2)
        super().__init__(**kw)


class Glm4MoeConfig(DecoderConfig):
    model_type = "glm4_moe"

    def __init__(self, **kw):
        kw.setdefault("partial_rotary_factor", 0.5)
        kw.setdefault("head_dim", 128)
        kw.setdefault("rms_norm_eps", 1e-5)
        kw.setdefault("scoring_func", "sigmoid")
        kw.setdefault("topk_method", "noaux_tc")
        kw.setdefault("n_shared_experts", 1)
        kw.setdefault("first_k_dense_replace", 1)
        kw.setdefault("attention_bias", True)
        kw.setdefault("norm_topk_prob", True)
        super().__init__(**kw)


class MistralConfig(DecoderConfig):
    """Llama architecture with optional sliding-window attention, which is expressed through the attention kernels' per-key
    "first masked row" bound (key j is masked from row j + window on)."""

    model_type = "mistral"

    def __init__(self, sliding_window=None, **kw):
        super().__init__(**kw)
        self.sliding_window = sliding_window


class Phi3Config(DecoderConfig):
    """Phi-3 / Phi-4: Llama blocks whose checkpoints already store the fused ``qkv_proj`` and ``gate_up_proj``
    matrices, which is this implementation's internal layout (paddleformers/transformers/phi3)."""

    model_type = "phi3"

    def __init__(self, sliding_window=None, **kw):
        kw.setdefault("rms_norm_eps", 1e-5)
        super().__init__(**kw)
        self.sliding_window = sliding_window
        self.hf_fused_qkv = True
        self.hf_fused_gate_up = True


class Glm4Config(DecoderConfig):
    """GLM-4 dense (paddleformers/transformers/glm_ocr text decoder, GLM-4-0414): a norm before and after both the attention
    and the MLP of every block, rotary embedding on the first half of each head with interleaved pairs in the checkpoint, fused
    ``gate_up_proj`` in the checkpoint."""

    model_type = "glm4"

    def __init__(self, **kw):
        kw.setdefault("partial_rotary_factor", 0.5)
        kw.setdefault("rms_norm_eps", 1e-5)
        super().__init__(**kw)
        self.block_style = "sandwich"
        self.hf_fused_gate_up = True
        self.rope_interleaved_checkpoint = True
        self.hf_name_translation = [["post_attention_layernorm", "post_self_attn_layernorm"],
                                    ["pre_feedforward_layernorm", "post_attention_layernorm"],
                                    ["post_feedforward_layernorm", "post_mlp_layernorm"]]

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            for k in ("block_style", "hf_fused_gate_up", "rope_interleaved_checkpoint", "hf_name_translation"):
                d.pop(k, None)
        return d


class SeedOssConfig(DecoderConfig):
    """Seed-OSS: Llama blocks with biases on q/k/v (paddleformers/transformers/seed_oss)."""

    model_type = "seed_oss"

    def __init__(self, attention_out_bias=False, **kw):
        kw.setdefault("attention_bias", True)
        super().__init__(**kw)
        self.attention_out_bias = bool(attention_out_bias)


class InternLM3Config(DecoderConfig):
    """InternLM3: Llama blocks; ``qkv_bias`` switches the q/k/v biases (paddleformers/transformers/internlm3)."""

    model_type = "internlm3"

    def __init__(self, qkv_bias=False, bias=False, **kw):
        kw.setdefault("attention_bias", bool(qkv_bias))
        kw.setdefault("mlp_bias", bool(bias))
        super().__init__(**kw)
        self.qkv_bias, self.bias = qkv_bias, bias
        self.attention_out_bias = bool(bias)


class HunYuanDenseV1Config(DecoderConfig):
    """Hunyuan dense: Llama blocks whose per-head QK RMSNorm runs AFTER the rotary embedding, and whose "dynamic" rotary rule
    with ``alpha`` is a plain change of base, theta * alpha ** (d / (d - 2)) (paddleformers/transformers/hunyuan)."""

    model_type = "hunyuan_v1_dense"

    def __init__(self, rope_parameters=None, **kw):
        kw.setdefault("rms_norm_eps", 1e-5)
        kw["use_qk_norm"] = True
        rp = dict(rope_parameters or {})
        alpha = rp.get("alpha") if rp.get("rope_type") == "dynamic" else None
        if alpha:
            rope_parameters = {"rope_type": "default", "rope_theta": rp.get("rope_theta", kw.get("rope_theta", 10000.0))}
        super().__init__(rope_parameters=rope_parameters, **kw)
        self.rope_alpha = float(alpha) if alpha else None
        if alpha:
            self.rope_base_theta = float(self.rope_theta)
            self.rope_theta = self.rope_base_theta * float(alpha) ** (self.head_dim / (self.head_dim - 2))
        self.qk_norm_after_rope = True
        self.qk_norm_hf_names = ("query_layernorm", "key_layernorm")
        self.attention_out_bias = bool(self.attention_bias)

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            if self.rope_alpha:
                d["rope_parameters"] = {"rope_type": "dynamic", "alpha": self.rope_alpha, "factor": 1.0, "rope_theta": self.rope_base_theta}
                d.pop("rope_theta", None)
            for k in ("rope_alpha", "rope_base_theta", "qk_norm_after_rope", "qk_norm_hf_names"):
                d.pop(k, None)
        return d


class HunYuanMoEV1Config(HunYuanDenseV1Config):
    """Hunyuan MoE: every layer routes with softmax top-k (renormalised) over experts of the dense width and adds one shared
    expert of the same width (paddleformers/transformers/hunyuan)."""

    model_type = "hunyuan_v1_moe"

    def __init__(self, moe_topk=1, num_experts=1, **kw):
        if not isinstance(num_experts, int) or not isinstance(moe_topk, int):
            raise NotImplementedError("per-layer expert counts / top-k lists are not implemented")
        kw.setdefault("num_experts_per_tok", moe_topk)
        kw.setdefault("norm_topk_prob", True)
        kw.setdefault("scoring_func", "softmax")
        kw.setdefault("n_shared_experts", 1)
        super().__init__(num_experts=num_experts, **kw)
        self.moe_topk = self.num_experts_per_tok
        self.moe_intermediate_size = self.moe_intermediate_size or self.intermediate_size
        self.shared_expert_intermediate_size = self.shared_expert_intermediate_size or self.intermediate_size
        self.shared_expert_hf_name = "shared_mlp"
        self.router_weight_hf_name = "gate.wg.weight"


class MixtralConfig(DecoderConfig):
    """Mixtral: Mistral attention (optional sliding window), every layer a softmax top-k router with renormalised weights over
    experts of the dense width; checkpoints name the block ``block_sparse_moe`` and the projections w1 / w3 / w2."""

    model_type = "mixtral"

    def __init__(self, sliding_window=None, **kw):
        kw.setdefault("norm_topk_prob", True)
        kw.setdefault("num_experts_per_tok", 2)
        kw.setdefault("router_aux_loss_coef", 0.001)
        kw.setdefault("rms_norm_eps", 1e-5)
        super().__init__(**kw)
        self.sliding_window = sliding_window
        self.moe_intermediate_size = self.moe_intermediate_size or self.intermediate_size
        self.moe_block_hf_name = "block_sparse_moe"
        self.expert_proj_hf_names = ("w1", "w3", "w2")
        self.num_local_experts = self.num_experts

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            d["num_local_experts"] = self.num_experts
            d.pop("num_experts", None)
        return d


class Qwen3NextConfig(DecoderConfig):
    """Qwen3-Next: three of four layers mix tokens with a gated delta-rule linear attention (``nn.linear_attention``), the
    fourth with softmax attention whose output is gated by a sigmoid computed from the query projection; rotary embedding on a
    quarter of each head, per-head QK norm, zero-centred RMSNorm weights ((1 + w), stored as w), MoE layers with a gated
    shared expert (paddleformers/transformers/qwen3_next). The linear-attention layers run as tensor operations."""

    model_type = "qwen3_next"

    def __init__(self, layer_types=None, full_attention_interval=4, linear_num_value_heads=32, linear_num_key_heads=16,
                 linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4, **kw):
        _expert_count_alias(kw)
        kw.setdefault("partial_rotary_factor", 0.25)
        kw.setdefault("use_qk_norm", True)
        kw.setdefault("head_dim", 256)
        kw.setdefault("norm_topk_prob", True)
        kw.setdefault("router_aux_loss_coef", 1e-3)
        if kw.get("num_experts") and kw.get("shared_expert_intermediate_size", 1):
            kw.setdefault("n_shared_experts", 1)
        super().__init__(**kw)
        n = self.num_hidden_layers
        self.full_attention_interval = full_attention_interval
        self.layer_types = list(layer_types) if layer_types else [
            "full_attention" if (i + 1) % full_attention_interval == 0 else "linear_attention" for i in range(n)]
        self.linear_num_value_heads, self.linear_num_key_heads = linear_num_value_heads, linear_num_key_heads
        self.linear_key_head_dim, self.linear_value_head_dim = linear_key_head_dim, linear_value_head_dim
        self.linear_conv_kernel_dim = linear_conv_kernel_dim
        self.attention_output_gate = True
        self.norm_weight_offset = 1.0
        self.shared_expert_gate = bool(self.n_shared_experts)
        self.shared_expert_hf_name = "shared_expert"

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            for k in ("attention_output_gate", "norm_weight_offset", "no_kv_cache", "shared_expert_gate", "shared_expert_hf_name"):
                d.pop(k, None)
        return d


class Qwen3_5TextConfig(Qwen3NextConfig):
    """Qwen3.5 (text decoder): Qwen3-Next's layer pattern with dense MLPs, four separate input projections in the
    linear-attention layers, and tensors stored under ``model.language_model`` because the released models are multimodal
    (paddleformers/transformers/qwen3_5). A multimodal configuration is reduced to its ``text_config``; the vision tower
    of the multimodal model is not provided."""

    model_type = "qwen3_5_text"

    def __init__(self, text_config=None, vision_config=None, **kw):
        if text_config:                                   # a multimodal config.json: keep the decoder's fields
            kw = {**{k: v for k, v in dict(text_config).items() if k != "model_type"},
                  **{k: v for k, v in kw.items() if k in ("tie_word_embeddings", "dtype", "torch_dtype", "architectures")}}
        rp = dict(kw.get("rope_parameters") or {})
        for k in ("mrope_section", "mrope_interleaved"):     # text-only use: the three position streams coincide
            rp.pop(k, None)
        if rp:
            kw["rope_parameters"] = rp
        super().__init__(**kw)
        self.linear_attn_split_projections = True
        self.hf_name_translation = [["model.", "model.language_model."]]

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            d.pop("linear_attn_split_projections", None)
            d.pop("hf_name_translation", None)
        return d


class Qwen3_5MoeTextConfig(Qwen3_5TextConfig):
    """Qwen3.5-MoE (text decoder): Qwen3.5 with Qwen3-Next's MoE layers (paddleformers/transformers/qwen3_5_moe)."""

    model_type = "qwen3_5_moe_text"


class Llama4TextConfig(DecoderConfig):
    """Llama 4 (text): local layers attend inside chunks of ``attention_chunk_size`` positions and rotate q / k (interleaved
    pairs in the checkpoint), followed by a weightless L2 norm of q and k; every ``no_rope_layer_interval``-th layer is global,
    uses no positional embedding and scales its queries with the logarithm of the position ("temperature tuning"). MoE layers
    (``moe_layers``) pick top-k experts by logit, multiply the expert INPUT by the sigmoid of that logit, and add a shared
    expert; dense layers use ``intermediate_size_mlp`` (paddleformers/transformers/llama4)."""

    model_type = "llama4_text"

    def __init__(self, intermediate_size_mlp=16384, attention_chunk_size=8192, layer_types=None, no_rope_layers=None,
                 no_rope_layer_interval=4, moe_layers=None, interleave_moe_layer_step=1, attn_temperature_tuning=True, attn_scale=0.1,
                 floor_scale=8192, use_qk_norm=True, **kw):
        kw.setdefault("num_experts_per_tok", 1)
        kw.setdefault("rms_norm_eps", 1e-5)
        kw.setdefault("rope_theta", 500000.0)
        kw.setdefault("n_shared_experts", 1)
        kw["scoring_func"] = "sigmoid_topk_logits"
        expert_size = kw.pop("intermediate_size", 8192)
        super().__init__(intermediate_size=intermediate_size_mlp, moe_intermediate_size=expert_size, use_qk_norm=False, **kw)
        n = self.num_hidden_layers
        self.intermediate_size_mlp, self.expert_intermediate_size = intermediate_size_mlp, expert_size
        self.shared_expert_intermediate_size = expert_size
        self.attention_chunk_size = attention_chunk_size
        self.no_rope_layer_interval = no_rope_layer_interval
        self.no_rope_layers = list(no_rope_layers) if no_rope_layers else [int((i + 1) % no_rope_layer_interval != 0) for i in range(n)]
        self.layer_types = list(layer_types) if layer_types else ["chunked_attention" if r else "full_attention" for r in self.no_rope_layers]
        self.interleave_moe_layer_step = interleave_moe_layer_step
        self.moe_layers = list(moe_layers) if moe_layers is not None else list(range(interleave_moe_layer_step - 1, n, interleave_moe_layer_step))
        self.attn_temperature_tuning, self.attn_scale, self.floor_scale = attn_temperature_tuning, attn_scale, floor_scale
        self.qk_l2_norm = bool(use_qk_norm)
        self.rope_interleaved_checkpoint = True
        self.moe_scale_expert_input = True
        self.hf_experts_style = "llama4"
        self.shared_expert_hf_name = "shared_expert"
        self.router_weight_hf_name = "router.weight"
        self.hf_name_translation = [[".mlp.", ".feed_forward."]]
        self.num_local_experts = self.num_experts

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            d["intermediate_size"] = self.expert_intermediate_size
            d["num_local_experts"] = self.num_experts
            d["use_qk_norm"] = self.qk_l2_norm
            for k in ("num_experts", "moe_intermediate_size", "scoring_func", "expert_intermediate_size", "qk_l2_norm",
                      "hf_experts_style", "hf_name_translation", "moe_scale_expert_input"):
                d.pop(k, None)
        return d


class GptOssConfig(DecoderConfig):
    """gpt-oss: attention with one learned sink logit per head, biases on all attention projections, alternating
    sliding-window and global layers, yarn rotary scaling; every layer routes with a biased router whose combine weights are a
    softmax over the selected logits, to experts with biases and a clamped gate (paddleformers/transformers/gpt_oss). Sinks
    and biased experts have no fused kernels here: attention runs in the eager back-end, the experts in tensor operations."""

    model_type = "gpt_oss"

    def __init__(self, sliding_window=128, layer_types=None, swiglu_limit=7.0, **kw):
        kw.setdefault("attention_bias", True)
        kw.setdefault("num_experts_per_tok", 4)
        kw.setdefault("rms_norm_eps", 1e-5)
        kw.setdefault("rope_theta", 150000.0)
        kw.setdefault("head_dim", 64)
        kw.setdefault("router_aux_loss_coef", 0.9)
        kw["scoring_func"] = "softmax_topk"
        super().__init__(**kw)
        self.sliding_window = sliding_window
        n = self.num_hidden_layers
        self.layer_types = list(layer_types) if layer_types else [
            "sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n)]
        self.swiglu_limit = swiglu_limit
        self.attention_out_bias = True
        self.attention_sinks = True
        self.router_bias = True
        self.expert_bias = True
        self.hf_experts_style = "gpt_oss"
        self.moe_intermediate_size = self.moe_intermediate_size or self.intermediate_size
        self.moe_token_dispatcher_type = "alltoall"
        self.num_local_experts = self.num_experts

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            d["num_local_experts"] = self.num_experts
            d.pop("num_experts", None)
            rp = {"rope_type": "default", **(self.rope_scaling or {}), "rope_theta": self.rope_theta}
            d["rope_parameters"] = rp
            for k in ("rope_theta", "rope_scaling", "scoring_func", "attention_sinks", "router_bias", "expert_bias", "hf_experts_style"):
                d.pop(k, None)
        return d


class DiffLlamaConfig(DecoderConfig):
    """Differential Transformer on Llama blocks: attention heads work in pairs and subtract a learned multiple of the second
    head's attention from the first (paddleformers/transformers/diff_transformer)."""

    model_type = "diffllama"

    def __init__(self, lambda_std_dev=0.1, **kw):
        kw.setdefault("rms_norm_eps", 1e-5)
        super().__init__(**kw)
        self.lambda_std_dev = lambda_std_dev
        self.differential_attention = True
        self.attention_out_bias = bool(self.attention_bias)
        self.no_kv_cache = True

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            for k in ("differential_attention", "no_kv_cache"):
                d.pop(k, None)
        return d


class MiniMaxConfig(MixtralConfig):
    """MiniMax-Text-01: Mixtral's MoE blocks, alternating softmax attention and fixed-decay "lightning" linear attention
    (``layer_types``), and a block whose residual stream continues from the normed input with per-branch alpha / beta factors
    (paddleformers/transformers/minimax)."""

    model_type = "minimax"

    def __init__(self, layer_types=None, block_size=256, full_attn_alpha_factor=1, full_attn_beta_factor=1, linear_attn_alpha_factor=1,
                 linear_attn_beta_factor=1, mlp_alpha_factor=1, mlp_beta_factor=1, **kw):
        kw.setdefault("rope_theta", 1000000.0)
        super().__init__(**kw)
        n = self.num_hidden_layers
        self.layer_types = list(layer_types) if layer_types else ["full_attention" if (i + 1) % 2 else "linear_attention" for i in range(n)]
        self.block_size = block_size
        self.full_attn_alpha_factor, self.full_attn_beta_factor = full_attn_alpha_factor, full_attn_beta_factor
        self.linear_attn_alpha_factor, self.linear_attn_beta_factor = linear_attn_alpha_factor, linear_attn_beta_factor
        self.mlp_alpha_factor, self.mlp_beta_factor = mlp_alpha_factor, mlp_beta_factor
        self.block_style = "normed_residual"
        self.linear_attention_kind = "lightning"

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            for k in ("block_style", "linear_attention_kind", "no_kv_cache"):
                d.pop(k, None)
        return d


class MiniMaxM2Config(DecoderConfig):
    """MiniMax-M2: one RMSNorm over all heads' query / key features before the rotary embedding, every layer a sigmoid
    router with a selection-only correction bias and renormalised top-k weights, experts of the dense width, no shared
    expert (paddleformers/transformers/minimax_m2)."""

    model_type = "minimax_m2"

    def __init__(self, **kw):
        kw.setdefault("scoring_func", "sigmoid")
        kw.setdefault("topk_method", "noaux_tc")
        kw.setdefault("norm_topk_prob", True)
        kw.setdefault("router_aux_loss_coef", 0.001)
        kw.setdefault("rope_theta", 5000000.0)
        super().__init__(**kw)
        self.qk_norm_full = True
        self.moe_intermediate_size = self.moe_intermediate_size or self.intermediate_size
        self.moe_block_hf_name = "block_sparse_moe"            # checkpoints use Mixtral's names: w1 = gate, w3 = up, w2 = down
        self.expert_proj_hf_names = ("w1", "w3", "w2")
        self.router_bias_name = "block_sparse_moe.e_score_correction_bias"
        self.router_bias_leading_dim = False
        self.num_local_experts = self.num_experts

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            d["num_local_experts"] = self.num_experts
            d.pop("num_experts", None)
        return d


class InternLM2Config(DecoderConfig):
    """InternLM2 / InternLM2.5: Llama blocks stored under their own names (``tok_embeddings``, ``attention.wqkv`` / ``wo``,
    ``feed_forward.w1`` / ``w3`` / ``w2``, ``attention_norm``, ``ffn_norm``, ``output``) with the fused ``wqkv`` rows grouped
    by kv head (paddleformers/transformers/intern_lm2, intern_lm2_5)."""

    model_type = "internlm2"

    def __init__(self, bias=False, **kw):
        if bias:
            raise NotImplementedError("InternLM2 checkpoints with projection biases are not handled")
        super().__init__(**kw)
        self.bias = False
        self.hf_fused_qkv = True
        self.qkv_grouped_by_kv_head = True
        self.hf_name_translation = [["model.embed_tokens.", "model.tok_embeddings."], ["lm_head.", "output."],
                                    ["self_attn.qkv_proj.", "attention.wqkv."], ["self_attn.o_proj.", "attention.wo."],
                                    ["input_layernorm.", "attention_norm."], ["post_attention_layernorm.", "ffn_norm."],
                                    ["mlp.gate_proj.", "feed_forward.w1."], ["mlp.up_proj.", "feed_forward.w3."],
                                    ["mlp.down_proj.", "feed_forward.w2."]]


class Qwen2MoeConfig(DecoderConfig):
    """Qwen2-MoE / Qwen1.5-MoE: softmax router without renormalisation, one wide shared expert whose output is gated per
    token by a sigmoid (paddleformers/transformers/qwen2_moe)."""

    model_type = "qwen2_moe"

    def __init__(self, **kw):
        _expert_count_alias(kw)
        kw.setdefault("attention_bias", True)
        kw.setdefault("num_experts", 60)
        kw.setdefault("num_experts_per_tok", 4)
        kw.setdefault("moe_intermediate_size", 1408)
        kw.setdefault("shared_expert_intermediate_size", 5632)
        kw.setdefault("n_shared_experts", 1)
        kw.setdefault("norm_topk_prob", False)
        kw.setdefault("router_aux_loss_coef", 1e-3)
        super().__init__(**kw)
        self.shared_expert_gate = True
        self.shared_expert_hf_name = "shared_expert"


class GraniteConfig(DecoderConfig):
    """Granite 3: Llama blocks with four scalar multipliers - on the embeddings, on every residual branch, as the
    attention softmax scale, and as a divisor of the logits (paddleformers/transformers/granite)."""

    model_type = "granite"

    def __init__(self, embedding_multiplier=1.0, residual_multiplier=1.0, attention_multiplier=None, logits_scaling=1.0, **kw):
        super().__init__(**kw)
        self.embedding_multiplier, self.residual_multiplier = float(embedding_multiplier), float(residual_multiplier)
        self.attention_multiplier = attention_multiplier
        self.logits_scaling = float(logits_scaling)


class MiniCPMConfig(GraniteConfig):
    """MiniCPM (muP-style scaling): embeddings x ``scale_emb``, every residual branch x ``scale_depth / sqrt(layers)``,
    hidden states / (hidden_size / dim_model_base) before the head (paddleformers/transformers/minicpm)."""

    model_type = "minicpm"

    def __init__(self, scale_emb=1.0, scale_depth=1.0, dim_model_base=None, **kw):
        L = int(kw.get("num_hidden_layers", 32))
        H = int(kw.get("hidden_size", 4096))
        kw.setdefault("embedding_multiplier", float(scale_emb))
        kw.setdefault("residual_multiplier", float(scale_depth) / (L ** 0.5))
        kw.setdefault("logits_scaling", float(H) / float(dim_model_base) if dim_model_base else 1.0)
        super().__init__(**kw)
        self.scale_emb, self.scale_depth, self.dim_model_base = scale_emb, scale_depth, dim_model_base


class MiniCPM4_1Config(MiniCPMConfig):
    """MiniCPM 4.1 (paddleformers/transformers/minicpm4_1): MiniCPM's scaling rules with long-rope frequency factors. The
    checkpoint's ``sparse_config`` describes a block-sparse key selection that the reference applies only to long prompts on
    the GPU; it is kept in the configuration and attention stays dense, which is exact up to ``sparse_config["dense_len"]``
    tokens and an approximation-free (more expensive) evaluation beyond it."""

    model_type = "minicpm4_1"

    def __init__(self, sparse_config=None, mup_denominator=32, **kw):
        kw.setdefault("tie_word_embeddings", True)
        super().__init__(**kw)
        self.sparse_config, self.mup_denominator = sparse_config, mup_denominator


class MiniCPM3Config(MiniCPMConfig):
    """MiniCPM3: MiniCPM's scaling rules on multi-head latent attention (low-rank q and kv projections, a rotary slice shared
    by all heads' keys) with half-split rotary pairs in the checkpoint and dense SwiGLU MLPs
    (paddleformers/transformers/minicpm3)."""

    model_type = "minicpm3"

    def __init__(self, qk_nope_head_dim=64, qk_rope_head_dim=32, q_lora_rank=768, kv_lora_rank=256, v_head_dim=None, **kw):
        kw.setdefault("tie_word_embeddings", True)
        kw["head_dim"] = qk_nope_head_dim + qk_rope_head_dim
        super().__init__(qk_nope_head_dim=qk_nope_head_dim, qk_rope_head_dim=qk_rope_head_dim, q_lora_rank=q_lora_rank,
                         kv_lora_rank=kv_lora_rank, v_head_dim=v_head_dim or qk_nope_head_dim, **kw)
        self.rope_interleave = False          # rotate_half convention: no row permutation on load
        self.num_key_value_heads = self.num_attention_heads


class Olmo2Config(DecoderConfig):
    """OLMo 2: normalisation AFTER each branch (x + norm(branch(x))) and one RMSNorm over all heads' query / key features
    (paddleformers/transformers/olmo2)."""

    model_type = "olmo2"

    def __init__(self, **kw):
        super().__init__(**kw)
        self.block_style, self.qk_norm_full = "post", True


class GemmaConfig(DecoderConfig):
    """Gemma (first generation): RMSNorm weights stored as (w - 1), GELU-gated MLP, embeddings scaled by sqrt(hidden),
    tied head (paddleformers/transformers/gemma)."""

    model_type = "gemma"

    def __init__(self, hidden_activation=None, **kw):
        kw.setdefault("tie_word_embeddings", True)
        kw.setdefault("head_dim", 256)
        kw["hidden_act"] = hidden_activation or kw.get("hidden_act") or "gelu_pytorch_tanh"
        if kw["hidden_act"] == "gelu":
            kw["hidden_act"] = "gelu_pytorch_tanh"          # the released checkpoints were trained with the tanh form
        super().__init__(**kw)
        self.hidden_activation = self.hidden_act
        self.embedding_multiplier = float(self.hidden_size) ** 0.5
        self.norm_weight_offset = 1.0


class Gemma2Config(GemmaConfig):
    """Gemma 2: Gemma with four norms per block, alternating sliding-window and global layers, a query scale of
    ``query_pre_attn_scalar ** -0.5`` and soft-capped attention scores and output logits. The flash kernels have no soft cap:
    attention runs in the eager back-end and the loss outside the fused head kernel (paddleformers/transformers lists the
    family through its Gemma support)."""

    model_type = "gemma2"

    def __init__(self, sliding_window=4096, layer_types=None, query_pre_attn_scalar=256, attn_logit_softcapping=50.0,
                 final_logit_softcapping=30.0, **kw):
        kw.setdefault("max_position_embeddings", 8192)
        super().__init__(**kw)
        self.sliding_window = sliding_window
        n = self.num_hidden_layers
        self.layer_types = list(layer_types) if layer_types else [
            "sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n)]
        self.query_pre_attn_scalar = query_pre_attn_scalar
        self.attention_multiplier = float(query_pre_attn_scalar) ** -0.5
        self.attn_logit_softcapping, self.final_logit_softcapping = attn_logit_softcapping, final_logit_softcapping
        self.block_style = "sandwich"

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            for k in ("attention_multiplier", "block_style"):
                d.pop(k, None)
        return d


class Gemma3TextConfig(GemmaConfig):
    """Gemma 3 (text): Gemma's (w - 1) norms, GeGLU and scaled embeddings, plus per-head QK norm, four norms per block (the
    branch output is normed before it joins the residual stream), a repeating pattern of sliding-window layers and global
    layers that use different rotary bases, and a query scale of ``query_pre_attn_scalar ** -0.5``
    (paddleformers/transformers/gemma3_text). Logit soft-capping, when a configuration sets it, takes the eager attention back-end like Gemma 2."""

    model_type = "gemma3_text"

    def __init__(self, sliding_window=4096, layer_types=None, sliding_window_pattern=6, query_pre_attn_scalar=256,
                 rope_local_base_freq=10000.0, rope_parameters=None, final_logit_softcapping=None, attn_logit_softcapping=None,
                 **kw):
        local_theta = float(rope_local_base_freq)
        if rope_parameters and "full_attention" in rope_parameters:      # recent Hugging Face configs: one entry per layer kind
            local_theta = float(rope_parameters.get("sliding_attention", {}).get("rope_theta", local_theta))
            rope_parameters = dict(rope_parameters["full_attention"])
        kw.setdefault("rope_theta", 1000000.0)
        kw.setdefault("use_qk_norm", True)
        kw.setdefault("max_position_embeddings", 131072)
        super().__init__(rope_parameters=rope_parameters, **kw)
        self.attn_logit_softcapping, self.final_logit_softcapping = attn_logit_softcapping, final_logit_softcapping
        self.sliding_window = sliding_window
        n = self.num_hidden_layers
        self.layer_types = list(layer_types) if layer_types else [
            "full_attention" if (i + 1) % int(sliding_window_pattern) == 0 else "sliding_attention" for i in range(n)]
        self.query_pre_attn_scalar = query_pre_attn_scalar
        self.attention_multiplier = float(query_pre_attn_scalar) ** -0.5
        self.rope_local_theta = local_theta
        self.block_style = "sandwich"

    def to_dict(self, saving: bool = False):
        d = super().to_dict(saving)
        if saving:
            full = {"rope_type": "default", "rope_theta": self.rope_theta}
            if self.rope_scaling:
                full = {**self.rope_scaling, "rope_theta": self.rope_theta}
            d["rope_parameters"] = {"sliding_attention": {"rope_type": "default", "rope_theta": self.rope_local_theta},
                                    "full_attention": full}
            for k in ("rope_theta", "rope_scaling", "rope_local_theta", "attention_multiplier", "block_style"):
                d.pop(k, None)
        return d


class CohereConfig(DecoderConfig):
    """Command-R: bias-free LayerNorm, attention and MLP in parallel on one normed input, interleaved rotary pairs in the
    checkpoint, logits multiplied by ``logit_scale`` (paddleformers/transformers/cohere)."""

    model_type = "cohere"

    def __init__(self, layer_norm_eps=1e-5, logit_scale=0.0625, **kw):
        kw.setdefault("rms_norm_eps", layer_norm_eps)
        kw.setdefault("tie_word_embeddings", True)
        super().__init__(**kw)
        self.layer_norm_eps, self.logit_scale = layer_norm_eps, logit_scale
        self.norm_type, self.block_style = "layernorm_nobias", "parallel"
        self.rope_interleaved_checkpoint = True
        self.logits_scaling = 1.0 / float(logit_scale)


class Cohere2Config(CohereConfig):
    """Command-R7B / Command-A: Cohere blocks with a repeating pattern of sliding-window layers, which rotate q and k, and
    global layers, which use no positional embedding at all (paddleformers/transformers/cohere2)."""

    model_type = "cohere2"

    def __init__(self, sliding_window=4096, layer_types=None, sliding_window_pattern=4, **kw):
        kw.setdefault("use_qk_norm", False)
        super().__init__(**kw)
        self.sliding_window = sliding_window
        n = self.num_hidden_layers
        self.layer_types = list(layer_types) if layer_types else [
            "full_attention" if (i + 1) % int(sliding_window_pattern) == 0 else "sliding_attention" for i in range(n)]
        self.rope_on_window_layers_only = True


class StableLmConfig(DecoderConfig):
    """StableLM 2: LayerNorm with bias, rotary embedding on the first quarter of each head, optional q/k/v biases
    (paddleformers/transformers/stablelm)."""

    model_type = "stablelm"

    def __init__(self, layer_norm_eps=1e-5, use_qkv_bias=False, **kw):
        kw.setdefault("rms_norm_eps", layer_norm_eps)
        kw.setdefault("attention_bias", bool(use_qkv_bias))
        kw.setdefault("partial_rotary_factor", 0.25)
        super().__init__(**kw)
        self.layer_norm_eps, self.use_qkv_bias = layer_norm_eps, use_qkv_bias
        self.norm_type = "layernorm"


class Ernie4_5Config(DecoderConfig):
    """ERNIE-4.5 dense: Llama blocks with tied embeddings whose checkpoints store q / k rows in the interleaved rotary
    order; the weight map permutes them to the half-split order on load and back on save
    (paddleformers/transformers/ernie4_5)."""

    model_type = "ernie4_5"

    def __init__(self, use_bias=False, **kw):
        kw.setdefault("rms_norm_eps", 1e-5)
        kw.setdefault("rope_theta", 500000.0)
        kw.setdefault("tie_word_embeddings", True)
        kw.setdefault("attention_bias", bool(use_bias))
        kw.setdefault("mlp_bias", bool(use_bias))
        super().__init__(**kw)
        self.use_bias = use_bias
        self.rope_interleaved_checkpoint = True


class Ernie4_5MoeConfig(Ernie4_5Config):
    """ERNIE-4.5 MoE (text): softmax router whose top-k selection adds a correction bias (``moe_statics``), weights
    renormalised over the selected experts, shared experts next to the routed ones, dense layers before
    ``moe_layer_start_index`` (paddleformers/transformers/ernie4_5_moe). The Hugging Face field names are accepted and
    translated."""

    model_type = "ernie4_5_moe"

    def __init__(self, moe_num_experts=None, moe_k=None, moe_num_shared_experts=None, moe_layer_start_index=None,
                 moe_layer_interval=None, moe_use_aux_free=True, moe_norm_min=1e-12, **kw):
        if moe_num_experts is not None:
            kw.setdefault("num_experts", int(moe_num_experts))
        if moe_k is not None:
            kw.setdefault("num_experts_per_tok", int(moe_k))
        if moe_num_shared_experts is not None:
            kw.setdefault("n_shared_experts", int(moe_num_shared_experts))
        if moe_layer_start_index is not None:
            kw.setdefault("first_k_dense_replace", int(moe_layer_start_index))
        if moe_layer_interval is not None:
            kw.setdefault("decoder_sparse_step", int(moe_layer_interval))
        kw.setdefault("scoring_func", "softmax")
        kw.setdefault("topk_method", "noaux_tc" if moe_use_aux_free else "greedy")
        kw.setdefault("norm_topk_prob", True)
        kw.setdefault("router_aux_loss_coef", 1e-3)
        super().__init__(**kw)
        self.moe_num_experts, self.moe_k = self.num_experts, self.num_experts_per_tok
        self.moe_num_shared_experts, self.moe_layer_start_index = self.n_shared_experts, self.first_k_dense_replace
        self.moe_layer_interval, self.moe_use_aux_free, self.moe_norm_min = self.decoder_sparse_step, moe_use_aux_free, moe_norm_min
        self.router_bias_name = "mlp.moe_statics.e_score_correction_bias"


CONFIG_MAPPING = {c.model_type: c for c in (Ernie4_5Config, Ernie4_5MoeConfig, Qwen2MoeConfig, GraniteConfig, MiniCPMConfig, Olmo2Config,
                                            GemmaConfig, Gemma2Config, Gemma3TextConfig, CohereConfig, Cohere2Config, StableLmConfig, LlamaConfig, Qwen2Config, Qwen3Config, Qwen3MoeConfig, DeepseekV3Config,
                                            Glm4MoeConfig, MistralConfig, Phi3Config, SeedOssConfig, InternLM3Config, HunYuanDenseV1Config,
                                            HunYuanMoEV1Config, MiniMaxM2Config, MixtralConfig, MiniCPM3Config, InternLM2Config, GptOssConfig, Llama4TextConfig, Qwen3NextConfig, Qwen3_5TextConfig, Qwen3_5MoeTextConfig, MiniMaxConfig, DiffLlamaConfig)}

# Families of the reference's registry (paddleformers/transformers/auto/modeling.py:55-112) whose blocks need a
# feature the unified decoder does not have; the Auto classes name the missing piece instead of failing on a key error.
UNSUPPORTED_FAMILIES = {
    # the reference holds a configuration and a checkpoint name map for these; the layers themselves come from its external
    # PaddleFleet package
    "deepseek_v4": "compressed sparse attention (the reference builds the layers from an external package)",
    "kimi_k3": "delta-rule linear attention with per-channel decay and block attention residuals (the reference builds the "
               "layers from an external package)",
    "hyperencoder": "an encoder stack of its own (the reference builds the layers from an external package)",
    # the reference ships processors only for these, and so does this package: transformers/kimi_processing.py (+
    # tool_declaration.py) and transformers/omni_processing.py
    "kimi_k25": "a vision tower (the reference ships its processor only; the processor is transformers.kimi_processing.KimiProcessor)",
    "qwen3_omni_moe": "audio / vision towers (the reference ships its processor only; the processor is "
                      "transformers.omni_processing.Qwen3OmniProcessor)",
}


# causal-LM families that are models of their own (not the unified decoder): model_type -> (module, config class, model class)
STANDALONE_FAMILIES = {
    "gemma4_text": ("gemma4", "Gemma4TextConfig", "Gemma4ForCausalLM"),
    "gemma4": ("gemma4", "Gemma4TextConfig", "Gemma4ForCausalLM"),          # the multimodal wrapper's text decoder
}


def _standalone(model_type: str, which: int):
    import importlib

    mod, *names = STANDALONE_FAMILIES[model_type]
    return getattr(importlib.import_module(f"{__package__}.{mod}"), names[which])


def resolve_config_class(model_type: str):
    if model_type in CONFIG_MAPPING:
        return CONFIG_MAPPING[model_type]
    if model_type in STANDALONE_FAMILIES:
        return _standalone(model_type, 0)
    if model_type in UNSUPPORTED_FAMILIES:
        raise NotImplementedError(f"model_type {model_type!r} is known but not implemented: it needs {UNSUPPORTED_FAMILIES[model_type]}")
    raise ValueError(f"unknown model_type {model_type!r}; supported: {sorted(CONFIG_MAPPING)}")
# families whose architecture is a strict subset of an implemented one load through it
CONFIG_MAPPING.update({"glm4": Glm4Config, "minicpm4_1": MiniCPM4_1Config, "qwen3_5": Qwen3_5TextConfig, "qwen3_5_moe": Qwen3_5MoeTextConfig, "kimi_k2": DeepseekV3Config, "deepseek_v2": DeepseekV2Config, "glm4_moe_lite": Glm4MoeLiteConfig, "glm_moe_dsa": GlmMoeDsaConfig, "deepseek_v32": DeepseekV32Config, "phi4": Phi3Config, "phi4flash": Phi3Config})


def named_config(name: str, **overrides) -> DecoderConfig:
    """Architecture presets used by the benchmark harness and tests (no checkpoint needed)."""
    presets = {
        "llama3-8b": (LlamaConfig, dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                                        num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=500000.0,
                                        rms_norm_eps=1e-5, max_position_embeddings=8192)),
        "qwen3-30b-a3b": (Qwen3MoeConfig, dict(vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                                               num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
                                               head_dim=128, num_experts=128, num_experts_per_tok=8,
                                               moe_intermediate_size=768, rope_theta=1e6, rms_norm_eps=1e-6,
                                               router_aux_loss_coef=1e-3, max_position_embeddings=40960)),
        "deepseek-v3-4l": (DeepseekV3Config, dict(num_hidden_layers=4, first_k_dense_replace=1, num_nextn_predict_layers=1)),
        "glm4.5-air-12l": (Glm4MoeConfig, dict(vocab_size=151552, hidden_size=4096, intermediate_size=10944,
                                               num_hidden_layers=12, num_attention_heads=96, num_key_value_heads=8,
                                               head_dim=128, n_routed_experts=128, num_experts_per_tok=8,
                                               moe_intermediate_size=1408, n_shared_experts=1, first_k_dense_replace=1,
                                               n_group=1, topk_group=1, routed_scaling_factor=1.0,
                                               num_nextn_predict_layers=1, rope_theta=1e6)),
        "tiny-llama": (LlamaConfig, dict(vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=2,
                                         num_attention_heads=4, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
                                         rope_theta=10000.0, max_position_embeddings=2048)),
    }
    cls, kw = presets[name]
    kw = dict(kw)
    kw.update(overrides)
    return cls(**kw)
