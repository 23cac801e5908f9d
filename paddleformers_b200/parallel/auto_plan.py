"""Automatic choice of the parallel degrees for a model on a given number of GPUs.

The reference offers a separate "auto-parallel" workflow built on a tracing compiler's sharding propagation
(paddleformers/cli/train/auto_parallel/workflow.py). Here the same user need - "I have N GPUs, make it fit and make it
fast" - is served by a small analytic planner over the hand-written strategies: it estimates per-GPU memory of every
candidate (sharding, expert, tensor, pipeline) combination from the model configuration and picks the cheapest one
that fits, preferring strategies in the order of their communication cost on an NVSwitch node:

1. optimizer-state sharding (one reduce-scatter + all-gather per step),
2. expert parallelism for MoE models (token exchange per MoE layer, experts are most of the weights),
3. tensor parallelism with sequence parallelism (two fused collectives per linear pair; inside one NVLink domain only),
4. pipeline parallelism (the only axis that should cross nodes; costs a bubble).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

from .topology import ParallelDegrees


@dataclass
class Plan:
    degrees: ParallelDegrees
    memory_gb: float
    breakdown: Dict[str, float]
    reason: str

    def training_args(self) -> Dict[str, object]:
        d = self.degrees
        out = {"tensor_model_parallel_size": d.mp, "pipeline_model_parallel_size": d.pp, "expert_model_parallel_size": d.ep,
               "sequence_parallel": d.mp > 1, "sharding": "stage1" if d.sharding > 1 else ""}
        if d.sharding > 1:
            out["sharding_parallel_size"] = d.sharding
        return out


def count_parameters(cfg) -> Dict[str, float]:
    """Dense (attention, dense MLPs, shared experts, norms, embeddings, head) and routed-expert parameter counts."""
    H, L = cfg.hidden_size, cfg.num_hidden_layers
    if cfg.is_mla:
        nh, qd = cfg.num_attention_heads, cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
        attn = (H * cfg.q_lora_rank + cfg.q_lora_rank * nh * qd) if cfg.q_lora_rank else H * nh * qd
        attn += H * (cfg.kv_lora_rank + cfg.qk_rope_head_dim) + cfg.kv_lora_rank * nh * (cfg.qk_nope_head_dim + cfg.v_head_dim)
        attn += nh * cfg.v_head_dim * H
    else:
        attn = H * (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim + cfg.num_attention_heads * cfg.head_dim * H
    dense = expert = 0.0
    n_mtp = int(getattr(cfg, "num_nextn_predict_layers", 0) or 0)
    for i in range(L + n_mtp):
        dense += attn + 2 * H
        if cfg.is_moe_layer(min(i, L - 1)):
            expert += cfg.num_experts * 3 * H * cfg.moe_intermediate_size
            dense += H * cfg.num_experts
            if cfg.n_shared_experts:
                dense += 3 * H * (cfg.shared_expert_intermediate_size or cfg.moe_intermediate_size * cfg.n_shared_experts)
        else:
            dense += 3 * H * cfg.intermediate_size
    emb = cfg.vocab_size * H
    dense += emb if getattr(cfg, "tie_word_embeddings", False) else 2 * emb
    return {"dense": dense, "expert": expert}


def activation_bytes_per_token(cfg, tp: int, recompute: bool) -> float:
    """Saved activations per token and layer in bf16 bytes (inputs of every GEMM, attention output and log-sum-exp,
    gate|up pre-activations); tensor parallel with sequence parallel divides all of it by tp. With full recompute only
    the layer input is kept."""
    H = cfg.hidden_size
    if recompute:
        return 2.0 * H / tp
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim if not cfg.is_mla else \
        cfg.num_attention_heads * (2 * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim) + cfg.v_head_dim)
    attn_out = cfg.num_attention_heads * (cfg.v_head_dim if cfg.is_mla else cfg.head_dim)
    if cfg.num_experts > 0:
        inter = cfg.moe_intermediate_size * cfg.num_experts_per_tok * 1.5   # capacity slack of the receive buffers
        mlp = 3 * inter + 2 * H * cfg.num_experts_per_tok
    else:
        mlp = 3 * cfg.intermediate_size
    return 2.0 * (4 * H + qkv + attn_out + mlp) / tp


def estimate_memory_gb(cfg, d: ParallelDegrees, seq_len: int, micro_batch: int = 1, recompute: bool = False,
                       in_flight_micro_batches: Optional[int] = None) -> Dict[str, float]:
    n = count_parameters(cfg)
    world_per_stage = d.world // d.pp
    dense_local = n["dense"] / (d.mp * d.pp)
    expert_local = n["expert"] / (d.ep * d.pp)
    moe_sharding = max(1, world_per_stage // d.ep)
    weights = 2.0 * (dense_local + expert_local)
    grads = 4.0 * (dense_local + expert_local)                      # fp32 main_grad
    opt = 12.0 * (dense_local / d.sharding + expert_local / (moe_sharding if d.ep > 1 else d.sharding))
    layers_local = cfg.num_hidden_layers / d.pp
    in_flight = in_flight_micro_batches if in_flight_micro_batches is not None else (d.pp if d.pp > 1 else 1)
    acts = activation_bytes_per_token(cfg, d.mp, recompute) * seq_len * micro_batch * layers_local * in_flight
    logits = 2048 * cfg.vocab_size / d.mp * 4.0 * 2                  # chunked head + cross entropy working set
    gib = float(1 << 30)
    out = {"weights": weights / gib, "grads": grads / gib, "optimizer": opt / gib, "activations": acts / gib,
           "loss_workspace": logits / gib, "runtime": 6.0}
    out["total"] = sum(out.values())
    return out


def _divisors(n: int) -> List[int]:
    return [i for i in range(1, n + 1) if n % i == 0]


def plan_parallelism(cfg, world_size: int, seq_len: int, micro_batch: int = 1, hbm_gb: float = 180.0,
                     gpus_per_node: int = 8, headroom: float = 0.9, recompute: bool = False) -> Plan:
    """Cheapest configuration (by the preference order of the module docstring) whose estimate fits in
    ``headroom * hbm_gb``. Raises if nothing fits even with every axis at its maximum."""
    budget = hbm_gb * headroom
    node = min(world_size, gpus_per_node)
    moe = cfg.num_experts > 0
    candidates = []
    for pp in _divisors(world_size):
        if cfg.num_hidden_layers % pp != 0 and pp > 1:
            continue
        per_stage = world_size // pp
        for tp in _divisors(min(per_stage, node)):
            if cfg.num_attention_heads % tp or cfg.num_key_value_heads % tp:
                continue
            rest = per_stage // tp
            eps = [e for e in _divisors(min(per_stage, node)) if cfg.num_experts % e == 0] if moe else [1]
            for ep in eps:
                if ep > 1 and tp > 1:
                    continue        # experts are not tensor-parallel in this framework: ep folds over the other axes
                d = ParallelDegrees(dp=1, sharding=rest, pp=pp, mp=tp, ep=ep)
                if d.world != world_size or per_stage % ep:
                    continue
                mem = estimate_memory_gb(cfg, d, seq_len, micro_batch, recompute)
                # cost: pipeline bubbles and cross-node traffic worst, then tensor parallel, then expert parallel
                cost = (pp - 1) * 100 + (tp - 1) * 10 + (0 if not moe else (node - ep))
                candidates.append((mem["total"] > budget, cost, mem["total"], d, mem))
    fitting = [c for c in candidates if not c[0]]
    if not fitting:
        best = min(candidates, key=lambda c: c[2])
        raise ValueError(f"no parallel configuration fits {budget:.0f} GB per GPU on {world_size} GPUs; the smallest estimate "
                         f"is {best[2]:.0f} GB with {best[3]} (try recompute or more GPUs)")
    _, cost, total, d, mem = min(fitting, key=lambda c: (c[1], c[2]))
    reason = (f"pp={d.pp} tp={d.mp} ep={d.ep} sharding={d.sharding}: estimated {total:.0f} GB of {hbm_gb:.0f} GB per GPU "
              f"(weights {mem['weights']:.0f}, grads {mem['grads']:.0f}, optimizer {mem['optimizer']:.0f}, activations "
              f"{mem['activations']:.0f})")
    return Plan(d, total, mem, reason)
