"""Gemma 4 text decoder, dense and mixture-of-experts (paddleformers/transformers/gemma4_moe/modeling.py:1-504,
configuration.py:20-136).

What sets the family apart from the unified decoder, and why it is a model of its own:

* head geometry per layer type: sliding-window layers use ``head_dim`` and ``num_key_value_heads``; full-attention layers
  use ``global_head_dim`` and, with ``attention_k_eq_v``, ``num_global_key_value_heads`` key heads whose (normed, unrotated)
  projection also serves as the value - those layers have no value projection;
* q and k are RMS-normed per head with a weight, v without one, and the score scale is 1;
* sliding layers rotate the whole head with their own base; full layers rotate only the first
  ``partial_rotary_factor`` of the frequency pairs ("proportional" rule: the remaining pairs get frequency zero);
* four norms per block; with ``enable_moe_block`` the feed-forward branch is the SUM of a dense gated MLP and a routed
  expert block, each behind its own post-norm, the experts reading the un-normed residual through their own pre-norm;
  the router norms its input without weights, scales it per channel and by 1/sqrt(hidden), takes a softmax over all
  experts, renormalises the k selected probabilities and multiplies them by a learned per-expert scale;
* per-layer input embeddings (a second, narrow embedding table per layer, mixed with a projection of the main embedding and
  gated into every block), layers that reuse the keys / values of the last earlier layer of their type
  (``num_kv_shared_layers``, optionally with a double-width MLP), a per-layer output scalar, and soft-capped final logits.

The routed experts go through the same dispatch plan / expert-parallel exchange as every other MoE layer of the package; their
activation is tanh-GELU, which the grouped SwiGLU kernels do not fuse, so they run segment by segment in tensor
operations. Attention runs through the flash kernel when a layer's head size is 128 and through the tensor-operation back-ends
otherwise (256 / 512-wide heads). Attention and the dense MLP are tensor parallel (column / row split, no sequence
parallelism); the routed experts are sharded by expert parallelism. Functional support, not a tuned path.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..generation.utils import GenerationMixin
from ..nn.attention import AttentionInterface
from ..nn.moe import GroupedExperts, _PermuteFn, build_dispatch_plan, unpermute_combine
from ..ops import functional as F
from ..parallel.topology import get_parallel_state
from ..transformers.configuration_utils import PretrainedConfig
from ..transformers.conversion_utils import Rule, WeightMap
from ..transformers.model_utils import PretrainedModel
from .modeling import CausalLMOutput, RMSNorm, _linear, _resolve_dtype

_ACT = {"gelu_pytorch_tanh": lambda x: TF.gelu(x, approximate="tanh"), "gelu": TF.gelu, "silu": TF.silu}


class Gemma4TextConfig(PretrainedConfig):
    model_type = "gemma4_text"
    is_mla = False
    no_kv_cache = True          # generation re-reads the prefix (the shared-kv layers make a per-layer cache a special case)

    def __init__(self, vocab_size=262144, hidden_size=2304, intermediate_size=9216, num_hidden_layers=30, num_attention_heads=8,
                 num_key_value_heads=4, head_dim=256, hidden_activation=None, hidden_act=None, max_position_embeddings=131072,
                 rms_norm_eps=1e-6, rope_parameters=None, attention_bias=False, sliding_window=512, layer_types=None,
                 final_logit_softcapping=None, vocab_size_per_layer_input=262144, hidden_size_per_layer_input=256,
                 num_global_key_value_heads=None, global_head_dim=512, attention_k_eq_v=False, num_kv_shared_layers=0,
                 enable_moe_block=False, use_double_wide_mlp=False, num_experts=None, top_k_experts=None,
                 moe_intermediate_size=None, interleaved_attn_pattern=None, sliding_window_rope_base=10000.0,
                 full_attention_rope_base=1000000.0, full_attention_rope_partial_factor=0.25, **kwargs):
        kwargs.setdefault("tie_word_embeddings", True)
        kwargs.setdefault("pad_token_id", 0)
        kwargs.setdefault("eos_token_id", 1)
        kwargs.setdefault("bos_token_id", 2)
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, num_hidden_layers=num_hidden_layers,
                         num_attention_heads=num_attention_heads, **kwargs)
        self.intermediate_size, self.num_key_value_heads, self.head_dim = intermediate_size, num_key_value_heads, head_dim
        self.hidden_activation = hidden_activation or hidden_act or "gelu_pytorch_tanh"
        self.max_position_embeddings, self.rms_norm_eps, self.attention_bias = max_position_embeddings, rms_norm_eps, attention_bias
        self.sliding_window, self.final_logit_softcapping = sliding_window, final_logit_softcapping
        self.vocab_size_per_layer_input, self.hidden_size_per_layer_input = vocab_size_per_layer_input, hidden_size_per_layer_input
        self.num_global_key_value_heads, self.global_head_dim = num_global_key_value_heads, global_head_dim
        self.attention_k_eq_v, self.num_kv_shared_layers = attention_k_eq_v, num_kv_shared_layers
        self.enable_moe_block, self.use_double_wide_mlp = enable_moe_block, use_double_wide_mlp
        self.num_experts, self.top_k_experts, self.moe_intermediate_size = num_experts, top_k_experts, moe_intermediate_size
        if layer_types is None:
            if interleaved_attn_pattern:              # (sliding, full) run lengths, the reference configuration's way to say it
                pat = ["sliding_attention"] * int(interleaved_attn_pattern[0]) + ["full_attention"] * int(interleaved_attn_pattern[1])
                layer_types = (pat * (num_hidden_layers // len(pat) + 1))[:num_hidden_layers]
            else:
                layer_types = ["sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(num_hidden_layers)]
        layer_types = list(layer_types)
        if layer_types:
            layer_types[-1] = "full_attention"          # the last layer always attends globally
        self.layer_types = layer_types
        if rope_parameters is None:
            rope_parameters = {"sliding_attention": {"rope_type": "default", "rope_theta": float(sliding_window_rope_base)},
                               "full_attention": {"rope_type": "proportional", "rope_theta": float(full_attention_rope_base),
                                                  "partial_rotary_factor": float(full_attention_rope_partial_factor)}}
        self.rope_parameters = rope_parameters

    @classmethod
    def from_dict(cls, d, **overrides):
        # released checkpoints carry the text model inside a multimodal wrapper configuration
        if d.get("model_type") == "gemma4" and "text_config" in d:
            d = d["text_config"]
        return super().from_dict(d, **overrides)

    # the package's generic MoE plumbing reads these names
    @property
    def num_experts_per_tok(self):
        return self.top_k_experts

    def layer_head_geometry(self, layer_idx: int):
        """(head size, key / value heads, keys double as values) of layer ``layer_idx``."""
        full = self.layer_types[layer_idx] != "sliding_attention"
        D = self.global_head_dim if (full and self.global_head_dim) else self.head_dim
        k_eq_v = bool(self.attention_k_eq_v and full)
        Hkv = self.num_global_key_value_heads if (k_eq_v and self.num_global_key_value_heads) else self.num_key_value_heads
        return D, Hkv, k_eq_v

    def kv_source_layer(self, layer_idx: int) -> Optional[int]:
        """Layer whose keys / values layer ``layer_idx`` reuses (the last unshared layer of the same type), or None."""
        first = self.num_hidden_layers - int(self.num_kv_shared_layers or 0)
        if not (layer_idx >= first > 0):
            return None
        prev = self.layer_types[:first]
        return len(prev) - 1 - prev[::-1].index(self.layer_types[layer_idx])


def rope_inverse_frequencies(params: dict, head_dim: int) -> torch.Tensor:
    """[head_dim / 2] rotation frequencies of one layer type. "default": base ** (-2i / D); "proportional": only the first
    ``partial_rotary_factor`` of the pairs rotate (same exponent, over the full head size), the others keep frequency zero."""
    base = float(params["rope_theta"])
    kind = params.get("rope_type", "default")
    if kind == "default":
        return 1.0 / base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)
    if kind != "proportional":
        raise NotImplementedError(f"rope_type {kind!r} for Gemma 4")
    n_rot = int(float(params.get("partial_rotary_factor", 1.0)) * head_dim // 2)
    inv = torch.zeros(head_dim // 2, dtype=torch.float32)
    inv[:n_rot] = 1.0 / base ** (torch.arange(0, 2 * n_rot, 2, dtype=torch.float32) / head_dim)
    return inv / float(params.get("factor", 1.0))


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of x [B, S, H, D] by cos / sin [B, S, D] (both halves carry the same angles)."""
    h = x.shape[-1] // 2
    rot = torch.cat([-x[..., h:], x[..., :h]], dim=-1)
    return x * cos[:, :, None, :] + rot * sin[:, :, None, :]


def _unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.pow(xf.pow(2).mean(-1, keepdim=True) + eps, -0.5)).to(x.dtype)


class Gemma4Attention(nn.Module):
    def __init__(self, config: Gemma4TextConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.D, self.Hkv, self.k_eq_v = config.layer_head_geometry(layer_idx)
        tp = get_parallel_state().degrees.mp
        assert config.num_attention_heads % tp == 0 and self.Hkv % tp == 0, \
            "Gemma 4: query heads and the key / value heads of every layer type must divide the tensor-parallel degree"
        self.Hq, self.Hkv = config.num_attention_heads // tp, self.Hkv // tp          # heads of this rank
        self.sliding = config.layer_types[layer_idx] == "sliding_attention"
        self.kv_source = config.kv_source_layer(layer_idx)
        self.eps = config.rms_norm_eps
        H, b, kw = config.hidden_size, bool(config.attention_bias), dict(dtype=dtype, device=device)
        self.q_proj = _linear(H, self.Hq * tp * self.D, b, "colwise", config, **kw)
        self.k_proj = _linear(H, self.Hkv * tp * self.D, b, "colwise", config, **kw)
        self.v_proj = None if self.k_eq_v else _linear(H, self.Hkv * tp * self.D, b, "colwise", config, **kw)
        self.o_proj = _linear(self.Hq * tp * self.D, H, b, "rowwise", config, **kw)
        self.q_norm = RMSNorm(self.D, self.eps, dtype=dtype, device=device)
        self.k_norm = RMSNorm(self.D, self.eps, dtype=dtype, device=device)
        if tp > 1:                 # shared by all heads, seen by this rank's heads only: partial gradients, summed over the group
            from ..parallel.tensor_parallel import mark_as_sequence_parallel_parameter

            mark_as_sequence_parallel_parameter(self.q_norm.weight)
            mark_as_sequence_parallel_parameter(self.k_norm.weight)
        self.impl = getattr(config, "_attn_implementation", None)

    def forward(self, x, cos, sin, kend, shared_kv: dict):
        B, S, _ = x.shape
        q = self.q_norm(self.q_proj(x).view(B, S, self.Hq, self.D))
        q = _rotate(q.float(), cos, sin).to(x.dtype)
        if self.kv_source is not None:
            k, v = shared_kv[self.kv_source]
        else:
            kr = self.k_proj(x).view(B, S, self.Hkv, self.D)
            vr = kr if self.v_proj is None else self.v_proj(x).view(B, S, self.Hkv, self.D)
            k = _rotate(self.k_norm(kr).float(), cos, sin).to(x.dtype)
            v = _unit_rms(vr, self.eps)
            shared_kv[self.layer_idx] = (k, v)
        if self.D == 128 and q.is_cuda and q.dtype == torch.bfloat16 and self.impl not in ("eager", "sdpa"):
            out = F.flash_attention(q.contiguous(), k.contiguous(), v.contiguous(), True, kend, 1.0)
        else:
            out = AttentionInterface.get(self.impl if self.impl in ("eager", "sdpa") else "sdpa")(q, k, v, kend, 1.0)
        return self.o_proj(out.reshape(B, S, self.Hq * self.D))


class Gemma4MLP(nn.Module):
    def __init__(self, config: Gemma4TextConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        wide = bool(config.use_double_wide_mlp) and config.kv_source_layer(layer_idx) is not None
        I = config.intermediate_size * (2 if wide else 1)
        kw = dict(dtype=dtype, device=device)
        self.gate_proj = _linear(config.hidden_size, I, False, "colwise", config, **kw)
        self.up_proj = _linear(config.hidden_size, I, False, "colwise", config, **kw)
        self.down_proj = _linear(I, config.hidden_size, False, "rowwise", config, **kw)
        self.act = _ACT[config.hidden_activation]

    def forward(self, x):
        return self.down_proj(self.act(self.gate_proj(x)) * self.up_proj(x))


class Gemma4Router(nn.Module):
    """(expert ids [T, k], combine weights [T, k]) from the un-normed residual stream."""

    def __init__(self, config: Gemma4TextConfig, dtype=None, device=None):
        super().__init__()
        self.k, self.eps = int(config.top_k_experts), config.rms_norm_eps
        self.root = config.hidden_size ** -0.5
        self.proj = nn.Linear(config.hidden_size, config.num_experts, bias=False, dtype=dtype, device=device)
        self.scale = nn.Parameter(torch.ones(config.hidden_size, dtype=dtype, device=device))
        self.per_expert_scale = nn.Parameter(torch.ones(config.num_experts, dtype=dtype, device=device))

    def forward(self, x2d):
        h = _unit_rms(x2d, self.eps) * self.scale * self.root
        probs = torch.softmax(self.proj(h), dim=-1)
        w, idx = torch.topk(probs, self.k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        return idx, w * self.per_expert_scale[idx]


class GeluGluExperts(GroupedExperts):
    """Stacked gated experts with a configurable activation: every run of 128-row blocks of one expert is two matrix products
    around ``act(gate) * up`` in tensor operations."""

    def __init__(self, config, dtype=None, device=None):
        super().__init__(config, dtype=dtype, device=device)
        self.act = _ACT[config.hidden_activation]
        self.use_fp8 = False

    def forward(self, rows, block_expert, counts=None, out=None, expert_rows=None, grad_rows_out=None):
        if out is not None or grad_rows_out is not None:
            raise NotImplementedError("GELU-gated experts take the all-to-all dispatcher (moe_token_dispatcher_type: alltoall)")
        be = block_expert.tolist()
        pieces, b = [], 0
        while b < len(be):
            e, b0 = be[b], b
            while b < len(be) and be[b] == e:
                b += 1
            seg = rows[b0 * 128:b * 128]
            if e < 0:
                pieces.append(torch.zeros_like(seg))
                continue
            g, u = TF.linear(seg, self.gate_up_proj[e]).chunk(2, -1)
            pieces.append(TF.linear(self.act(g) * u, self.down_proj[e]))
        return torch.cat(pieces, dim=0) if pieces else torch.zeros_like(rows)


class Gemma4MoeBlock(nn.Module):
    """Router + routed experts of one layer; ``experts`` / ``config`` are what the expert-parallel exchange reads."""

    def __init__(self, config: Gemma4TextConfig, dtype=None, device=None):
        super().__init__()
        self.config = config
        self.router = Gemma4Router(config, dtype=dtype, device=device)
        self.experts = GeluGluExperts(config, dtype=dtype, device=device)
        self.ep = get_parallel_state().degrees.ep

    def forward(self, routed_from2d, x2d):
        idx, w = self.router(routed_from2d)
        if self.ep > 1:
            from ..parallel.expert_parallel import ep_moe_forward

            return ep_moe_forward(self, x2d, idx, w)
        dest, block_expert, rows, counts = build_dispatch_plan(idx, self.experts.num_local, 0)
        yr = self.experts(_PermuteFn.apply(x2d, dest, idx.shape[1], rows), block_expert, counts)
        return unpermute_combine(yr, dest, w, x2d.shape[0])


class Gemma4DecoderLayer(nn.Module):
    def __init__(self, config: Gemma4TextConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        H, eps, kw = config.hidden_size, config.rms_norm_eps, dict(dtype=dtype, device=device)
        self.self_attn = Gemma4Attention(config, layer_idx, **kw)
        self.mlp = Gemma4MLP(config, layer_idx, **kw)
        for nm in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            setattr(self, nm, RMSNorm(H, eps, **kw))
        self.register_buffer("layer_scalar", torch.ones(1, **kw))
        self.ple = int(config.hidden_size_per_layer_input or 0)
        if self.ple:
            self.act = _ACT[config.hidden_activation]
            self.per_layer_input_gate = nn.Linear(H, self.ple, bias=False, **kw)
            self.per_layer_projection = nn.Linear(self.ple, H, bias=False, **kw)
            self.post_per_layer_input_norm = RMSNorm(H, eps, **kw)
        self.moe = None
        if config.enable_moe_block:
            self.moe = Gemma4MoeBlock(config, **kw)
            for nm in ("post_feedforward_layernorm_1", "post_feedforward_layernorm_2", "pre_feedforward_layernorm_2"):
                setattr(self, nm, RMSNorm(H, eps, **kw))

    def forward(self, x, per_layer_input, cos, sin, kend, shared_kv):
        x = x + self.post_attention_layernorm(self.self_attn(self.input_layernorm(x), cos, sin, kend, shared_kv))
        h = self.mlp(self.pre_feedforward_layernorm(x))
        if self.moe is not None:
            flat = x.reshape(-1, x.shape[-1])
            routed = self.moe(flat, self.pre_feedforward_layernorm_2(flat)).reshape(x.shape)
            h = self.post_feedforward_layernorm_1(h) + self.post_feedforward_layernorm_2(routed)
        x = x + self.post_feedforward_layernorm(h)
        if self.ple:
            g = self.act(self.per_layer_input_gate(x)) * per_layer_input
            x = x + self.post_per_layer_input_norm(self.per_layer_projection(g))
        return x * self.layer_scalar


class Gemma4TextModel(nn.Module):
    def __init__(self, config: Gemma4TextConfig, dtype=None, device=None):
        super().__init__()
        self.config = config
        kw = dict(dtype=dtype, device=device)
        H, L = config.hidden_size, config.num_hidden_layers
        self.layer_range = range(L)
        self.embed_tokens = nn.Embedding(config.vocab_size, H, **kw)
        self.layers = nn.ModuleList([Gemma4DecoderLayer(config, i, **kw) for i in range(L)])
        self.norm = RMSNorm(H, config.rms_norm_eps, **kw)
        self.ple = int(config.hidden_size_per_layer_input or 0)
        if self.ple:
            self.embed_tokens_per_layer = nn.Embedding(config.vocab_size_per_layer_input, L * self.ple, **kw)
            self.per_layer_model_projection = nn.Linear(H, L * self.ple, bias=False, **kw)
            self.per_layer_projection_norm = RMSNorm(self.ple, config.rms_norm_eps, **kw)
        for lt in set(config.layer_types):
            D = config.global_head_dim if (lt != "sliding_attention" and config.global_head_dim) else config.head_dim
            self.register_buffer(f"inv_freq_{lt}", rope_inverse_frequencies(config.rope_parameters[lt], D).to(device), persistent=False)

    def per_layer_inputs(self, input_ids, embeds):
        """[B, S, L, P]: (normed projection of the main embedding + the token's per-layer embedding) / sqrt(2)."""
        cfg, L = self.config, self.config.num_hidden_layers
        proj = self.per_layer_model_projection(embeds) * cfg.hidden_size ** -0.5
        proj = self.per_layer_projection_norm(proj.reshape(*embeds.shape[:-1], L, self.ple))
        # the scale is rounded to the weights' dtype first, as the checkpoint's own implementation does
        tok = self.embed_tokens_per_layer(input_ids) * torch.tensor(self.ple ** 0.5, dtype=embeds.dtype, device=embeds.device)
        return (proj + tok.reshape(*input_ids.shape, L, self.ple)) * 2.0 ** -0.5

    def forward(self, input_ids, position_ids=None, kend=None):
        cfg = self.config
        B, S = input_ids.shape
        x = self.embed_tokens(input_ids)
        x = x * torch.tensor(cfg.hidden_size ** 0.5, dtype=x.dtype, device=x.device)
        ple = self.per_layer_inputs(input_ids, x) if self.ple else None
        pos = position_ids if position_ids is not None else torch.arange(S, device=x.device)[None].expand(B, -1)
        j = torch.arange(S, device=x.device, dtype=torch.int32)[None].expand(B, -1)
        doc_end = kend.to(torch.int32) if kend is not None else None
        win = j + int(cfg.sliding_window)                  # key j is hidden from query rows >= j + window
        kend_local = torch.minimum(win, doc_end) if doc_end is not None else win
        tables = {}
        for lt in set(cfg.layer_types):
            ang = pos[..., None].float() * getattr(self, f"inv_freq_{lt}").float()
            ang = torch.cat([ang, ang], dim=-1)
            tables[lt] = (ang.cos(), ang.sin())
        shared_kv = {}
        for i, layer in enumerate(self.layers):
            lt = cfg.layer_types[i]
            cos, sin = tables[lt]
            x = layer(x, ple[:, :, i] if ple is not None else None, cos, sin,
                      kend_local if lt == "sliding_attention" else doc_end, shared_kv)
        return self.norm(x)


class Gemma4ForCausalLM(PretrainedModel, GenerationMixin):
    config_class = Gemma4TextConfig
    base_model_prefix = "model"

    def __init__(self, config: Gemma4TextConfig, dtype=None, device=None):
        super().__init__(config)
        assert not (get_parallel_state().degrees.mp > 1 and getattr(config, "sequence_parallel", False)), \
            "Gemma 4: tensor parallelism without sequence parallelism"
        dtype = dtype if dtype is not None else _resolve_dtype(config.dtype)
        self.model = Gemma4TextModel(config, dtype=dtype, device=device)
        self.lm_head = None if config.tie_word_embeddings else \
            nn.Linear(config.hidden_size, config.vocab_size, bias=False, dtype=dtype, device=device)
        self.ignore_index = -100
        self.loss_accumulation_steps = 1
        self.post_init()

    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, (nn.Linear, nn.Embedding)):
            nn.init.normal_(module.weight, 0.0, std)
            if getattr(module, "bias", None) is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, GroupedExperts):
            nn.init.normal_(module.gate_up_proj, 0.0, std)
            nn.init.normal_(module.down_proj, 0.0, std)

    def head_weight(self):
        return self.model.embed_tokens.weight if self.lm_head is None else self.lm_head.weight

    def compute_logits(self, hidden):
        logits = TF.linear(hidden, self.head_weight())
        cap = self.config.final_logit_softcapping
        return torch.tanh(logits / cap) * cap if cap else logits

    def forward(self, input_ids, labels=None, position_ids=None, attn_mask_startend_row_indices=None, kend=None, caches=None,
                return_logits: Optional[bool] = None, **unused):
        """``labels`` are next-token targets aligned with ``input_ids``; ``attn_mask_startend_row_indices`` / ``kend``: int
        [B, S], key column j is hidden from query rows >= kend[j] (packed documents)."""
        assert caches is None, "Gemma 4 decodes by re-reading the prefix"
        if kend is None and attn_mask_startend_row_indices is not None:
            kend = attn_mask_startend_row_indices.reshape(input_ids.shape[0], -1)
        hidden = self.model(input_ids, position_ids, kend)
        out = CausalLMOutput()
        if return_logits if return_logits is not None else labels is None:
            out.logits = self.compute_logits(hidden)
        if labels is not None:
            lab, h2 = labels.reshape(-1), hidden.reshape(-1, hidden.shape[-1])
            count = (lab != self.ignore_index).sum()
            total = h2.new_zeros((), dtype=torch.float32)
            for lo in range(0, h2.shape[0], 2048):              # only a slice of the [tokens, vocabulary] logits is alive at a time
                total = total + TF.cross_entropy(self.compute_logits(h2[lo:lo + 2048]).float(), lab[lo:lo + 2048],
                                                 ignore_index=self.ignore_index, reduction="sum")
            out.loss = total / (count.clamp(min=1) * float(self.loss_accumulation_steps))
            out.num_tokens = count
        return out

    def weight_map(self) -> WeightMap:
        """Tensor names are the checkpoint's own, except the router / experts, which sit under ``moe.`` here."""
        rules = []
        for name, _ in list(self.named_parameters()) + [(n, None) for n, _ in self.named_buffers() if n.endswith("layer_scalar")]:
            rules.append(Rule(name, [name.replace(".moe.router.", ".router.").replace(".moe.experts.", ".experts.")]))
        return WeightMap(rules)

    def get_hardware_flops_per_token(self, seq_len: int) -> float:
        cfg = self.config
        dense = sum(p.numel() for n, p in self.named_parameters() if "embed_tokens" not in n and ".experts." not in n)
        if cfg.enable_moe_block:
            dense += cfg.num_hidden_layers * cfg.top_k_experts * 3 * cfg.hidden_size * cfg.moe_intermediate_size
        attn = 0
        for i in range(cfg.num_hidden_layers):
            D, _, _ = cfg.layer_head_geometry(i)
            span = min(seq_len, cfg.sliding_window) if cfg.layer_types[i] == "sliding_attention" else seq_len
            attn += 2 * 2 * cfg.num_attention_heads * D * span / 2
        return 3.0 * (2.0 * (dense + cfg.vocab_size * cfg.hidden_size) + attn)
