"""Model FLOPs per token (forward + backward = 3x forward), used for the TFLOPs / MFU columns of the training log.

Counts matmul FLOPs of the attention projections (GQA or MLA), causal-halved attention scores, the active experts
(+ shared experts), dense MLPs, the MTP layers and the logits, like the reference's DeepSeek-V3 model
(paddleformers/transformers/deepseek_v3/mfu_utils.py:132-190) generalised to every family of the zoo.
"""
from __future__ import annotations


def _attn_flops(cfg, S: int) -> float:
    H = cfg.hidden_size
    if cfg.is_mla:
        nh, qd, vd = cfg.num_attention_heads, cfg.qk_nope_head_dim + cfg.qk_rope_head_dim, cfg.v_head_dim
        proj = 0
        if cfg.q_lora_rank:
            proj += H * cfg.q_lora_rank + cfg.q_lora_rank * nh * qd
        else:
            proj += H * nh * qd
        proj += H * (cfg.kv_lora_rank + cfg.qk_rope_head_dim) + cfg.kv_lora_rank * nh * (cfg.qk_nope_head_dim + vd)
        proj += nh * vd * H
        core = nh * (qd + vd) * S / 2  # causal: half of the S x S score matrix
        return 2 * proj + 2 * core
    D = cfg.head_dim
    proj = H * (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * D + cfg.num_attention_heads * D * H
    core = cfg.num_attention_heads * 2 * D * S / 2
    return 2 * proj + 2 * core


def _mlp_flops(cfg, layer_idx: int) -> float:
    H = cfg.hidden_size
    if cfg.is_moe_layer(layer_idx):
        I = cfg.moe_intermediate_size
        f = 2 * 3 * H * I * cfg.num_experts_per_tok + 2 * H * cfg.num_experts
        if cfg.n_shared_experts:
            si = cfg.shared_expert_intermediate_size or I * cfg.n_shared_experts
            f += 2 * 3 * H * si
        return f
    return 2 * 3 * H * cfg.intermediate_size


def model_flops_per_token(cfg, seq_len: int, include_backward: bool = True) -> float:
    fwd = 0.0
    for i in range(cfg.num_hidden_layers):
        fwd += _attn_flops(cfg, seq_len) + _mlp_flops(cfg, i)
    n_mtp = int(getattr(cfg, "num_nextn_predict_layers", 0) or 0)
    for k in range(n_mtp):
        i = cfg.num_hidden_layers + k
        moe_like = cfg.num_experts > 0
        fwd += _attn_flops(cfg, seq_len) + (_mlp_flops(cfg, cfg.first_k_dense_replace) if moe_like else _mlp_flops(cfg, -1))
        fwd += 2 * 2 * cfg.hidden_size * cfg.hidden_size  # eh_proj
        fwd += 2 * cfg.hidden_size * cfg.vocab_size
    fwd += 2 * cfg.hidden_size * cfg.vocab_size
    return fwd * (3.0 if include_backward else 1.0)
