"""Unified decoder-only transformer covering the Llama / Qwen2 / Qwen3 / Qwen3-MoE / DeepSeek-V3 / GLM-4.5 families.

One implementation, configured by ``DecoderConfig``: GQA or MLA attention, optional per-head QK RMSNorm, full or
partial rotary embedding, dense SwiGLU or MoE feed-forward (softmax / sigmoid routers, shared experts, leading dense
layers) and multi-token-prediction (MTP) layers. Activations are kept 2-D ``[tokens, hidden]`` between blocks (token
sharded when sequence parallel is on), exactly one fused qkv and one fused gate|up projection per layer, residual
adds fused into the RMSNorm kernels.

Reference behaviour reproduced: paddleformers/transformers/llama/modeling.py:71-642 (attention, decoder layer,
causal LM), qwen3_moe/modeling.py:116-392 (QK-norm attention, sparse block), deepseek_v3/modeling.py:341-1128 (router,
MLA, MTP layer), glm4_moe/modeling.py:135-385 (partial rope, router) and the criterion's loss normalisation
(paddleformers/nn/criterion/sft_loss.py:44-57).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.utils.checkpoint

from ..nn.moe import DenseMLP, MoELayer
from ..generation.utils import GenerationMixin
from ..ops import functional as F
from ..utils.refined_recompute import checkpoint_keeping, keep, kept_ops_of_layer
from ..parallel.tensor_parallel import (AllGatherOp, ColumnParallelLinear, CopyToTP, GatherLastDimOp, GatherOp, RowParallelLinear, ScatterOp,
                                        VocabParallelEmbedding, mark_as_sequence_parallel_parameter)
from ..parallel.topology import get_parallel_state
from ..transformers.conversion_utils import Rule, WeightMap, expand_layers
from ..transformers.model_utils import PretrainedModel
from .configuration import (DecoderConfig, DeepseekV3Config, Glm4MoeConfig, InternLM3Config, LlamaConfig, MistralConfig,
                            Phi3Config, Qwen2Config, Qwen3Config, Qwen3MoeConfig, SeedOssConfig, Ernie4_5Config, Ernie4_5MoeConfig,
                            GraniteConfig, MiniCPMConfig, MiniCPM4_1Config, Glm4Config, Qwen2MoeConfig, Olmo2Config, GemmaConfig, Gemma2Config, Gemma3TextConfig, CohereConfig, Cohere2Config, StableLmConfig,
                            HunYuanDenseV1Config, HunYuanMoEV1Config, MiniMaxM2Config, MixtralConfig, MiniCPM3Config, InternLM2Config, GptOssConfig, Llama4TextConfig, Qwen3NextConfig, Qwen3_5TextConfig, Qwen3_5MoeTextConfig, GlmMoeDsaConfig, DeepseekV32Config, MiniMaxConfig, DiffLlamaConfig)


@dataclass
class BatchContext:
    """Per-forward metadata shared by all layers."""

    B: int
    S: int
    positions: Optional[torch.Tensor]   # [B*S] position ids (None = arange per sequence)
    kend: Optional[torch.Tensor]        # [B, S] int32 document mask bounds (None = plain causal)
    cos: torch.Tensor
    sin: torch.Tensor
    cp_positions: Optional[torch.Tensor] = None   # context parallel: global positions of the local tokens
    S_full: int = 0                               # context / segment parallel: length of the whole sequence
    kend_full: Optional[torch.Tensor] = None      # [B, S_full] document bounds of all keys (cp / sep)
    kend_window: Optional[torch.Tensor] = None    # [B, S] bounds of sliding-window layers: min(kend, key index + window)
    window: int = 0
    cos_local: Optional[torch.Tensor] = None      # rotary tables of sliding-window layers when they use their own base
    sin_local: Optional[torch.Tensor] = None
    kstart: Optional[torch.Tensor] = None         # [B, S] first row that sees key j (blocks with two-way attention); None = causal


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None
    aux_loss: Optional[torch.Tensor] = None
    mtp_losses: Optional[List[torch.Tensor]] = None
    num_tokens: Optional[torch.Tensor] = None
    past_key_values: Optional[object] = None


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float, sequence_parallel: bool = False, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.eps = eps
        if sequence_parallel:
            mark_as_sequence_parallel_parameter(self.weight)

    def forward(self, x, residual=None):
        return F.rms_norm(x, self.weight, self.eps, residual=residual)


class LayerNormAdapter(nn.Module):
    """LayerNorm (optionally without bias) behind the call convention of ``RMSNorm``: ``norm(x)`` or
    ``norm(x, residual) -> (normed(x + residual), x + residual)``. Statistics are computed in fp32."""

    def __init__(self, hidden_size: int, eps: float, bias: bool = True, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=device)) if bias else None
        self.eps = eps

    def _ln(self, x):
        y = torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), None, None, self.eps) * self.weight.float()
        if self.bias is not None:
            y = y + self.bias.float()
        return y.to(x.dtype)

    def forward(self, x, residual=None):
        if residual is None:
            return self._ln(x)
        s = x + residual
        return self._ln(s), s


def make_norm(config, hidden_size: int, sequence_parallel: bool = False, dtype=None, device=None):
    """RMSNorm (fused kernel) unless the family asks for LayerNorm (``norm_type``: rms | layernorm | layernorm_nobias)."""
    kind = getattr(config, "norm_type", "rms") or "rms"
    if kind == "rms":
        return RMSNorm(hidden_size, config.rms_norm_eps, sequence_parallel, dtype=dtype, device=device)
    assert get_parallel_state().degrees.mp == 1, "LayerNorm families are implemented for tensor-parallel degree 1"
    return LayerNormAdapter(hidden_size, config.rms_norm_eps, bias=kind == "layernorm", dtype=dtype, device=device)


def _linear(in_f, out_f, bias, tp_plan, config, sections=None, dtype=None, device=None):
    """Linear factory with a tensor-parallel plan ("colwise" | "rowwise" | None), like the reference's
    ``Linear.create(..., tp_plan=...)`` (paddleformers/nn/linear.py:39-59)."""
    tp = get_parallel_state().degrees.mp
    sp = bool(getattr(config, "sequence_parallel", False))
    if tp > 1 and tp_plan == "colwise":
        return ColumnParallelLinear(in_f, out_f, bias=bias, sections=sections, sequence_parallel=sp, dtype=dtype, device=device)
    if tp > 1 and tp_plan == "rowwise":
        return RowParallelLinear(in_f, out_f, bias=bias, sequence_parallel=sp, dtype=dtype, device=device)
    return nn.Linear(in_f, out_f, bias=bias, dtype=dtype, device=device)


def _apply(mod, x):
    if isinstance(mod, nn.Linear):
        return F.linear(x, mod.weight, mod.bias)
    return mod(x)


def long_sequence_attention(q, k, v, ctx: "BatchContext", scale: float, config) -> Optional[torch.Tensor]:
    """Attention when the sequence is split over ranks. q, k, v: [B, S_local, H, D].

    * context parallel (``cp`` axis): keys / values are all-gathered over the group and the local queries attend by
      global position (``context_parallel_algo = "ring"`` selects the K/V ring instead, plain causal masks only);
    * Ulysses (``sep`` axis): all-to-all to [B, S, H / sep, D], ordinary attention on whole sequences, all-to-all back
      (paddleformers/transformers/segment_parallel_utils.py:69-137).

    Returns None when neither axis is active."""
    ps = get_parallel_state()
    if ps.degrees.cp > 1 and ctx.cp_positions is not None:
        from ..parallel.context_parallel import cp_attention, ring_attention

        mode = getattr(config, "cp_balance_mode", None) or "dualchunk_allgather"
        if getattr(config, "context_parallel_algo", "allgather") == "ring" and ctx.kend_full is None:
            return ring_attention(q, k, v, ps.group("cp"), ctx.S_full, mode, scale)
        return cp_attention(q, k, v, ctx.cp_positions, ctx.S_full, mode, ps.group("cp"), scale, ctx.kend_full)
    if ps.degrees.sep > 1:
        from ..parallel.context_parallel import ReshardLayer

        n, g = ps.degrees.sep, ps.group("sep")
        assert q.shape[2] % n == 0, "segment parallel needs the query heads (per tensor-parallel rank) to divide sep"
        if k.shape[2] % n != 0:     # fewer key/value heads than ranks: replicate them so that every rank owns one
            rep = n // math.gcd(n, k.shape[2])
            k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
        qh, kh, vh = (ReshardLayer.apply(t.contiguous(), g, True) for t in (q, k, v))
        out = F.flash_attention(qh, kh, vh, True, ctx.kend_full if ctx.kend_full is not None else None, scale)
        return ReshardLayer.apply(out.contiguous(), g, False)
    return None


class Attention(nn.Module):
    """GQA attention with a fused qkv projection laid out as [q heads | k heads | v heads]."""

    def __init__(self, config: DecoderConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        tp = get_parallel_state().degrees.mp
        self.config = config
        self.D = config.head_dim
        self.Hq_total, self.Hkv_total = config.num_attention_heads, config.num_key_value_heads
        assert self.Hq_total % tp == 0 and self.Hkv_total % tp == 0, "heads must divide the tensor parallel degree"
        self.Hq, self.Hkv = self.Hq_total // tp, self.Hkv_total // tp
        self.rot = int(self.D * config.partial_rotary_factor)
        H = config.hidden_size
        secs = [self.Hq_total * self.D, self.Hkv_total * self.D, self.Hkv_total * self.D]
        # attention_output_gate (Qwen3-Next): the query projection also produces one gate value per output feature, stored per
        # head as [q | gate]; the attention output is multiplied by sigmoid(gate). Such layers keep q / k / v projections apart.
        self.output_gate = bool(getattr(config, "attention_output_gate", False))
        if self.output_gate:
            assert tp == 1, "gated attention is implemented for tensor-parallel degree 1"
            self.q_proj = nn.Linear(H, 2 * secs[0], bias=config.attention_bias, dtype=dtype, device=device)
            self.k_proj = nn.Linear(H, secs[1], bias=config.attention_bias, dtype=dtype, device=device)
            self.v_proj = nn.Linear(H, secs[2], bias=config.attention_bias, dtype=dtype, device=device)
            self.qkv_proj = None
        else:
            self.qkv_proj = _linear(H, sum(secs), config.attention_bias, "colwise", config, sections=secs, dtype=dtype, device=device)
        self.o_proj = _linear(self.Hq_total * self.D, H, bool(getattr(config, "attention_out_bias", False)), "rowwise", config,
                              dtype=dtype, device=device)
        self.use_qk_norm = config.use_qk_norm
        self.clip_qkv = float(getattr(config, "clip_qkv", 0.0) or 0.0)          # projections clamped to [-c, c] (Molmo / OLMo)
        self.qk_norm_full = bool(getattr(config, "qk_norm_full", False))      # one RMSNorm over all heads' features (OLMo2)
        if self.qk_norm_full:
            assert tp == 1, "full-width QK norm is implemented for tensor-parallel degree 1"
            self.use_qk_norm = False
            self.q_norm = RMSNorm(self.Hq * self.D, config.rms_norm_eps, dtype=dtype, device=device)
            self.k_norm = RMSNorm(self.Hkv * self.D, config.rms_norm_eps, dtype=dtype, device=device)
        elif self.use_qk_norm:
            self.q_norm = RMSNorm(self.D, config.rms_norm_eps, dtype=dtype, device=device)
            self.k_norm = RMSNorm(self.D, config.rms_norm_eps, dtype=dtype, device=device)
            if tp > 1:
                # one weight vector shared by all heads, but every tensor-parallel rank sees its own heads only: the
                # gradients are partial sums and are added up over the group before the optimizer step
                mark_as_sequence_parallel_parameter(self.q_norm.weight)
                mark_as_sequence_parallel_parameter(self.k_norm.weight)
        self.qk_norm_after_rope = bool(self.use_qk_norm and getattr(config, "qk_norm_after_rope", False))   # Hunyuan
        self.scale = float(getattr(config, "attention_multiplier", None) or 1.0 / math.sqrt(self.D))
        # soft-capped attention scores and attention sinks are not in the flash kernels: such families run the eager back-end
        self.softcap = float(getattr(config, "attn_logit_softcapping", None) or 0.0)
        self.sinks = nn.Parameter(torch.zeros(self.Hq, dtype=dtype, device=device)) if getattr(config, "attention_sinks", False) else None
        if self.sinks is not None and tp > 1:
            self.sinks.shard_spec = ("tp", 0, None)
        self.window = config.layer_window(layer_idx)
        self.local_rope = bool(self.window and getattr(config, "rope_local_theta", None))
        # families whose global layers carry no positional embedding (Cohere2): only window layers rotate
        self.use_rope = bool(self.window) or not getattr(config, "rope_on_window_layers_only", False)
        # Llama 4: chunked local layers; listed layers without rotary embedding; a weightless L2 norm of q and k after the
        # rotation on the rotating layers; position-dependent query scale on the others
        # differential attention (DiffLlama): heads work in pairs (j, j + H/2); the pair's output is softmax_j V - lambda *
        # softmax_{j+H/2} V on a value twice as wide (both halves' values side by side), RMS-normalised without weights
        self.differential = bool(getattr(config, "differential_attention", False))
        if self.differential:
            assert tp == 1 and self.Hq % 2 == 0, "differential attention: even head count, tensor-parallel degree 1"
            std = float(getattr(config, "lambda_std_dev", 0.1))
            for nm in ("lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2"):
                setattr(self, nm, nn.Parameter(torch.randn(self.D, dtype=dtype, device=device) * std))
            self.lambda_init = 0.8 - 0.6 * math.exp(-0.3 * layer_idx)
        self.chunk = config.layer_chunk(layer_idx)
        nope = getattr(config, "no_rope_layers", None)
        if nope is not None and layer_idx < len(nope):
            self.use_rope = bool(nope[layer_idx])
        self.qk_l2 = bool(getattr(config, "qk_l2_norm", False)) and self.use_rope
        self.temp_tuning = bool(getattr(config, "attn_temperature_tuning", False)) and not self.use_rope

    def forward(self, x2d: torch.Tensor, ctx: BatchContext, cache=None) -> torch.Tensor:
        gate = None
        if self.output_gate:
            qg = _apply(self.q_proj, x2d).view(x2d.shape[0], self.Hq, 2 * self.D)
            gate = qg[..., self.D:].reshape(x2d.shape[0], self.Hq * self.D)
            qkv = torch.cat([qg[..., :self.D].reshape(x2d.shape[0], self.Hq * self.D), _apply(self.k_proj, x2d), _apply(self.v_proj, x2d)], dim=-1)
        else:
            qkv = keep("attention_column_ln", _apply, self.qkv_proj, x2d)
        if self.clip_qkv:
            qkv = qkv.clamp(-self.clip_qkv, self.clip_qkv)
        kend = ctx.kend_window if ((self.window or self.chunk) and ctx.kend_window is not None) else ctx.kend
        cos, sin = (ctx.cos_local, ctx.sin_local) if (self.local_rope and ctx.cos_local is not None) else (ctx.cos, ctx.sin)
        if self.qk_norm_full:
            nq, nk = self.Hq * self.D, self.Hkv * self.D
            qkv = torch.cat([self.q_norm(qkv[:, :nq].contiguous()), self.k_norm(qkv[:, nq:nq + nk].contiguous()), qkv[:, nq + nk:]], dim=-1)
        if self.qk_norm_after_rope:
            qkv = F.rope_packed(qkv, cos, sin, ctx.positions, self.Hq, self.Hkv, self.D, self.rot)
            nq, nk = self.Hq * self.D, self.Hkv * self.D
            qn = self.q_norm(qkv[:, :nq].reshape(-1, self.D)).reshape(-1, nq)
            kn = self.k_norm(qkv[:, nq:nq + nk].reshape(-1, self.D)).reshape(-1, nk)
            qkv = torch.cat([qn, kn, qkv[:, nq + nk:]], dim=-1)
        elif self.use_qk_norm:
            qkv = F.qk_norm_rope_packed(qkv, self.q_norm.weight, self.k_norm.weight, cos, sin, ctx.positions,
                                        self.Hq, self.Hkv, self.D, self.rot, self.config.rms_norm_eps)
        elif self.use_rope:
            qkv = F.rope_packed(qkv, cos, sin, ctx.positions, self.Hq, self.Hkv, self.D, self.rot)
        if self.qk_l2 or self.temp_tuning:
            nq, nk = self.Hq * self.D, self.Hkv * self.D
            q, k = qkv[:, :nq], qkv[:, nq:nq + nk]
            if self.qk_l2:
                eps = self.config.rms_norm_eps

                def l2(t):
                    t = t.reshape(-1, self.D).float()
                    return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)).reshape(x2d.shape[0], -1)

                q, k = l2(q).to(qkv.dtype), l2(k).to(qkv.dtype)
            if self.temp_tuning:
                pos = ctx.positions if ctx.positions is not None else torch.arange(ctx.S, device=qkv.device).repeat(ctx.B)
                sc = torch.log1p(torch.floor((pos.float() + 1.0) / float(self.config.floor_scale))) * float(self.config.attn_scale) + 1.0
                q = (q.float() * sc[:, None]).to(qkv.dtype)
            qkv = torch.cat([q, k, qkv[:, nq + nk:]], dim=-1)
        if self.differential:
            if cache is not None or ctx.S_full:
                raise NotImplementedError("differential attention: no incremental cache, no context / segment parallelism")
            B, S, D, half = ctx.B, ctx.S, self.D, self.Hq // 2
            rep = self.Hq // self.Hkv
            q, k, v = qkv.view(B, S, -1).split([self.Hq * D, self.Hkv * D, self.Hkv * D], dim=-1)
            q = q.reshape(B, S, self.Hq, D)
            k = k.reshape(B, S, self.Hkv, D).repeat_interleave(rep, dim=2)
            v = v.reshape(B, S, self.Hkv, D).repeat_interleave(rep, dim=2)
            v2 = torch.cat([v[:, :, :half], v[:, :, half:]], dim=-1).repeat(1, 1, 2, 1)          # [B, S, Hq, 2D]
            o = F.flash_attention(q, k.contiguous(), v2.contiguous(), True, kend, self.scale)
            lam = torch.exp((self.lambda_q1.float() * self.lambda_k1.float()).sum()) \
                - torch.exp((self.lambda_q2.float() * self.lambda_k2.float()).sum()) + self.lambda_init
            o = o[:, :, :half].float() - lam * o[:, :, half:].float()
            o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.config.rms_norm_eps) * (1.0 - self.lambda_init)
            return _apply(self.o_proj, o.to(x2d.dtype).reshape(B * S, self.Hq * D))
        if cache is not None:
            out = cache.attend(self, qkv, ctx)
        elif (self.softcap or self.sinks is not None or ctx.kstart is not None
              or getattr(self.config, "_attn_implementation", None) in ("eager", "sdpa")) and not ctx.S_full:
            from ..nn.attention import AttentionInterface      # reference back-ends, selectable like the reference's

            B, S, D = ctx.B, ctx.S, self.D
            q, k, v = qkv.view(B, S, -1).split([self.Hq * D, self.Hkv * D, self.Hkv * D], dim=-1)
            impl = "eager" if (self.softcap or self.sinks is not None) else (getattr(self.config, "_attn_implementation", None) or "sdpa")
            impl = impl if impl in ("eager", "sdpa") else "sdpa"
            extra = {"softcap": self.softcap} if self.softcap else {}
            if ctx.kstart is not None:                    # two-way blocks: the flash kernels take the upper bound only
                extra["kstart"] = ctx.kstart
            if self.sinks is not None:
                extra["sinks"] = self.sinks
            out = AttentionInterface.get(impl)(
                q.reshape(B, S, self.Hq, D), k.reshape(B, S, self.Hkv, D), v.reshape(B, S, self.Hkv, D), kend, self.scale, **extra)
            out = out.reshape(B * S, self.Hq * D)
        elif self.softcap or self.sinks is not None or ctx.kstart is not None:
            raise NotImplementedError("soft-capped scores / attention sinks / two-way blocks are not combined with context / segment parallelism")
        elif ctx.S_full:
            B, S, D = ctx.B, ctx.S, self.D
            q, k, v = qkv.view(B, S, -1).split([self.Hq * D, self.Hkv * D, self.Hkv * D], dim=-1)
            out = long_sequence_attention(q.reshape(B, S, self.Hq, D), k.reshape(B, S, self.Hkv, D),
                                          v.reshape(B, S, self.Hkv, D), ctx, self.scale, self.config)
            out = out.reshape(B * S, self.Hq * D)
        else:
            out = keep("flash_attn", F.flash_attention_qkvpacked, qkv, ctx.B, ctx.S, self.Hq, self.Hkv, self.D, True, kend, self.scale)
        if gate is not None:
            out = out * torch.sigmoid(gate.float()).to(out.dtype)
        return keep("attention_row_ln", _apply, self.o_proj, out)


class SparseIndexer(nn.Module):
    """Token selector of DeepSeek sparse attention (DSA): a light multi-head scorer, score[s, t] = sum_h w[s, h] *
    relu(q[s, h] . k[t]) / sqrt(d), with its own projections (queries from the latent query, one shared key per token, rotary
    embedding on the first ``qk_rope_head_dim`` features in half-split order) picks the ``index_topk`` keys a query may attend
    to (paddleformers/transformers/deepseek_v32, glm_moe_dsa). Selection is not differentiated through."""

    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.H, self.D, self.rope = config.index_n_heads, config.index_head_dim, config.qk_rope_head_dim
        self.topk = int(config.index_topk)
        self.wq_b = nn.Linear(config.q_lora_rank, self.H * self.D, bias=False, **kw)
        self.wk = nn.Linear(config.hidden_size, self.D, bias=False, **kw)
        self.k_norm = nn.LayerNorm(self.D, eps=1e-6, **kw)
        self.weights_proj = nn.Linear(config.hidden_size, self.H, bias=False, **kw)

    @torch.no_grad()
    def visible(self, x2d, q_latent, ctx: "BatchContext", allowed: torch.Tensor) -> torch.Tensor:
        """allowed: bool [B, S, S] (causal / document mask). Returns bool [B, S, S]: the selected keys among the allowed ones."""
        B, S = ctx.B, ctx.S
        T = B * S
        q = self.wq_b(q_latent).view(T, self.H, self.D)
        k = self.k_norm(self.wk(x2d))
        q_pe = F.rope_heads(q[..., :self.rope].reshape(T, self.H * self.rope), ctx.cos, ctx.sin, ctx.positions, self.H, self.rope)
        k_pe = F.rope_heads(k[:, :self.rope].contiguous(), ctx.cos, ctx.sin, ctx.positions, 1, self.rope)
        q = torch.cat([q_pe.view(T, self.H, self.rope), q[..., self.rope:]], dim=-1).view(B, S, self.H, self.D)
        k = torch.cat([k_pe.view(T, self.rope), k[:, self.rope:]], dim=-1).view(B, S, self.D)
        w = self.weights_proj(x2d).float().view(B, S, self.H) * self.H ** -0.5
        sc = torch.relu(torch.einsum("bshd,btd->bsht", q.float(), k.float()) * self.D ** -0.5)
        score = torch.einsum("bsht,bsh->bst", sc, w).masked_fill(~allowed, float("-inf"))
        idx = score.topk(min(self.topk, S), dim=-1).indices
        return torch.zeros_like(allowed).scatter_(-1, idx, True) & allowed


class MLAAttention(nn.Module):
    """Multi-head latent attention (DeepSeek-V3), non-absorbed training form: low-rank q and kv projections with
    RMSNorm on the latents, rotary embedding on a separate ``qk_rope_head_dim`` slice whose key part is shared by
    all heads, q/k head dim = nope + rope, v head dim separate
    (paddleformers/transformers/deepseek_v3/modeling.py:542-801)."""

    def __init__(self, config: DecoderConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        tp = get_parallel_state().degrees.mp
        self.config = config
        H = config.hidden_size
        self.Hq_total = config.num_attention_heads
        self.Hq = self.Hq_total // tp
        self.nope, self.rope, self.vd = config.qk_nope_head_dim, config.qk_rope_head_dim, config.v_head_dim
        self.qd = self.nope + self.rope
        self.q_lora, self.kv_lora = config.q_lora_rank, config.kv_lora_rank
        if self.q_lora:
            self.q_a_proj = nn.Linear(H, self.q_lora, bias=False, dtype=dtype, device=device)
            self.q_a_layernorm = RMSNorm(self.q_lora, config.rms_norm_eps, dtype=dtype, device=device)
            self.q_b_proj = _linear(self.q_lora, self.Hq_total * self.qd, False, "colwise", config, dtype=dtype, device=device)
        else:
            self.q_proj = _linear(H, self.Hq_total * self.qd, False, "colwise", config, dtype=dtype, device=device)
        self.kv_a_proj_with_mqa = nn.Linear(H, self.kv_lora + self.rope, bias=False, dtype=dtype, device=device)
        self.kv_a_layernorm = RMSNorm(self.kv_lora, config.rms_norm_eps, dtype=dtype, device=device)
        self.kv_b_proj = _linear(self.kv_lora, self.Hq_total * (self.nope + self.vd), False, "colwise", config, dtype=dtype, device=device)
        self.o_proj = _linear(self.Hq_total * self.vd, H, False, "rowwise", config, dtype=dtype, device=device)
        self.scale = 1.0 / math.sqrt(self.qd)
        rs = config.rope_scaling
        if rs and rs.get("mscale_all_dim"):
            m = 0.1 * float(rs["mscale_all_dim"]) * math.log(float(rs.get("factor", 1.0))) + 1.0
            self.scale = self.scale * m * m
        self.tp = tp
        self.sp = bool(getattr(config, "sequence_parallel", False)) and tp > 1
        self.group = get_parallel_state().group("mp")
        if self.sp:
            # the replicated low-rank projections and their norms see this rank's token slice only: partial gradients,
            # summed over the group before the optimizer step
            reps = [self.kv_a_proj_with_mqa.weight, self.kv_a_layernorm.weight]
            reps += [self.q_a_proj.weight, self.q_a_layernorm.weight] if self.q_lora else []
            for p in reps:
                mark_as_sequence_parallel_parameter(p)
        self.indexer = None
        if getattr(config, "index_topk", None):
            assert tp == 1 and self.q_lora, "sparse (indexer) attention needs the latent query and tensor-parallel degree 1"
            self.indexer = SparseIndexer(config, dtype=dtype, device=device)

    def forward(self, x2d, ctx: BatchContext, cache=None):
        T = ctx.B * ctx.S
        qa = None
        if self.q_lora:
            qa = self.q_a_layernorm(_apply(self.q_a_proj, x2d))
            q = _apply(self.q_b_proj, qa)
        else:
            q = _apply(self.q_proj, x2d)
        ckv = _apply(self.kv_a_proj_with_mqa, x2d)
        kv_lat, k_pe = ckv[:, : self.kv_lora], ckv[:, self.kv_lora:]
        # the latent goes through a column-parallel projection, which gathers token slices (sequence parallelism) and sums
        # the heads' gradients over the ranks itself; the shared rotary key does not, so it gets the same treatment here:
        # every rank's heads read it, and their gradients are added up on the way back
        kv = _apply(self.kv_b_proj, self.kv_a_layernorm(kv_lat.contiguous()))
        if self.tp > 1:
            k_pe = AllGatherOp.apply(k_pe.contiguous(), self.group) if self.sp else CopyToTP.apply(k_pe.contiguous(), self.group)
        q = q.view(T, self.Hq, self.qd)
        kv = kv.view(T, self.Hq, self.nope + self.vd)
        q_pe = F.rope_heads(q[..., self.nope:].reshape(T, self.Hq * self.rope), ctx.cos, ctx.sin, ctx.positions,
                            self.Hq, self.rope).view(T, self.Hq, self.rope)
        k_pe = F.rope_heads(k_pe.contiguous(), ctx.cos, ctx.sin, ctx.positions, 1, self.rope).view(T, 1, self.rope)
        qf = torch.cat([q[..., : self.nope], q_pe], dim=-1)
        kf = torch.cat([kv[..., : self.nope], k_pe.expand(T, self.Hq, self.rope)], dim=-1)
        v = kv[..., self.nope:]
        q4, k4 = qf.view(ctx.B, ctx.S, self.Hq, self.qd), kf.view(ctx.B, ctx.S, self.Hq, self.qd)
        v4 = v.reshape(ctx.B, ctx.S, self.Hq, self.vd)
        if self.indexer is not None and ctx.S > self.indexer.topk:
            # more keys than the selector keeps: every query attends to its selected keys only. The mask is arbitrary per
            # query, which the flash kernels cannot express: scores and softmax run as tensor operations here.
            if ctx.S_full:
                raise NotImplementedError("sparse (indexer) attention is not combined with context / segment parallelism")
            from ..nn.attention import _dense_mask

            allowed = _dense_mask(ctx.kend, ctx.B, ctx.S, True, x2d.device)
            vis = self.indexer.visible(x2d, qa, ctx, allowed)
            sc = torch.einsum("bshd,bthd->bhst", q4.float(), k4.float()) * self.scale
            p = torch.softmax(sc.masked_fill(~vis[:, None], float("-inf")), dim=-1)
            out = torch.einsum("bhst,bthd->bshd", p, v4.float()).to(x2d.dtype)
        elif ctx.S_full and cache is None:
            out = long_sequence_attention(q4, k4, v4, ctx, self.scale, self.config)
        else:
            out = F.flash_attention(q4, k4, v4, True, ctx.kend, self.scale)
        return _apply(self.o_proj, out.reshape(T, self.Hq * self.vd))


class DecoderLayer(nn.Module):
    def __init__(self, config: DecoderConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        sp = bool(getattr(config, "sequence_parallel", False)) and get_parallel_state().degrees.mp > 1
        self.layer_idx = layer_idx
        # block_style: "pre" (norm -> branch -> add, the default), "post" (branch -> norm -> add: OLMo2) or "parallel"
        # (attention and MLP read the same normed input and are added together: Cohere)
        # or "sandwich" (norm -> branch -> norm -> add, four norms per block: Gemma 3)
        self.block_style = getattr(config, "block_style", "pre") or "pre"
        # or "normed_residual" (MiniMax-Text: the residual stream continues from the NORMED input, x <- a * norm(x) + b * branch)
        if self.block_style == "normed_residual":
            self.input_layernorm = make_norm(config, config.hidden_size, sp, dtype=dtype, device=device)
            self.post_attention_layernorm = make_norm(config, config.hidden_size, sp, dtype=dtype, device=device)
            lin = bool(getattr(config, "layer_types", None)) and config.layer_types[layer_idx] == "linear_attention"
            self.attn_ab = (float(getattr(config, "linear_attn_alpha_factor" if lin else "full_attn_alpha_factor", 1.0)),
                            float(getattr(config, "linear_attn_beta_factor" if lin else "full_attn_beta_factor", 1.0)))
            self.mlp_ab = (float(getattr(config, "mlp_alpha_factor", 1.0)), float(getattr(config, "mlp_beta_factor", 1.0)))
        elif self.block_style == "sandwich":
            for nm in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
                setattr(self, nm, make_norm(config, config.hidden_size, sp, dtype=dtype, device=device))
        elif self.block_style != "parallel":
            self.input_layernorm = make_norm(config, config.hidden_size, sp, dtype=dtype, device=device) \
                if self.block_style == "pre" else None
            self.post_attention_layernorm = make_norm(config, config.hidden_size, sp, dtype=dtype, device=device)
            if self.block_style == "post":
                self.post_feedforward_layernorm = make_norm(config, config.hidden_size, sp, dtype=dtype, device=device)
        else:
            self.input_layernorm = make_norm(config, config.hidden_size, sp, dtype=dtype, device=device)
        attn_cls = MLAAttention if config.is_mla else Attention
        types = getattr(config, "layer_types", None)
        if types and layer_idx < len(types) and types[layer_idx] == "linear_attention":
            from ..nn.linear_attention import GatedDeltaNet, LightningAttention

            # a linear-attention token mixer instead of softmax attention: gated delta rule (Qwen3-Next) or fixed-decay
            # "lightning" attention (MiniMax-Text); called like an attention module
            mixer = LightningAttention if getattr(config, "linear_attention_kind", "gated_delta") == "lightning" else GatedDeltaNet
            self.linear_attn = mixer(config, layer_idx, dtype=dtype, device=device)
            self.self_attn = self.linear_attn.forward
        else:
            self.self_attn = attn_cls(config, layer_idx, dtype=dtype, device=device)
        if config.is_moe_layer(layer_idx) and getattr(config, "moe_modality_isolated", False):
            from ..nn.moe import ModalityMoELayer

            self.mlp = ModalityMoELayer(config, dtype=dtype, device=device)
        elif config.is_moe_layer(layer_idx):
            self.mlp = MoELayer(config, dtype=dtype, device=device)
        else:
            self.mlp = DenseMLP(config.hidden_size, config.intermediate_size, config, bias=config.mlp_bias, dtype=dtype, device=device)
        # recompute_granularity="selective": recompute_modules names the sub-modules ("attn", "mlp") whose activations are
        # dropped and rebuilt in the backward pass (paddleformers/transformers/configuration_utils.py:264-283)
        mods = getattr(config, "recompute_modules", None) or []
        if isinstance(mods, str):
            mods = [m.strip() for m in mods.split(",") if m.strip()]
        alias = {"self_attn": "attn", "attention": "attn", "core_attn": "attn", "moe": "mlp", "experts": "mlp"}
        self._selective = tuple(sorted({alias.get(m, m) for m in mods})) \
            if getattr(config, "recompute_granularity", None) == "selective" else ()
        self.residual_multiplier = float(getattr(config, "residual_multiplier", 1.0) or 1.0)

    def forward(self, hidden, residual, ctx: BatchContext, cache=None):
        """(branch output, residual stream) in, (branch output, residual stream) out; the add happens inside the
        next RMSNorm kernel."""
        if self.block_style != "pre":
            x = hidden if residual is None else hidden + residual
            if self.block_style == "normed_residual":
                h = self.input_layernorm(x)
                x = h * self.attn_ab[0] + self.self_attn(h, ctx, cache) * self.attn_ab[1]
                h = self.post_attention_layernorm(x)
                return h * self.mlp_ab[0] + self.mlp(h) * self.mlp_ab[1], None
            if self.block_style == "sandwich":
                x = x + self.post_attention_layernorm(self.self_attn(self.input_layernorm(x), ctx, cache))
                return x + self.post_feedforward_layernorm(self.mlp(self.pre_feedforward_layernorm(x))), None
            if self.block_style == "post":
                x = x + self.post_attention_layernorm(self.self_attn(x, ctx, cache))
                return x + self.post_feedforward_layernorm(self.mlp(x)), None
            normed = self.input_layernorm(x)
            return x + self.self_attn(normed, ctx, cache) + self.mlp(normed), None
        if residual is None:
            normed, residual = self.input_layernorm(hidden), hidden
        else:
            normed, residual = self.input_layernorm(hidden, residual)
        sel = self._selective if (self.training and cache is None) else ()
        if "attn" in sel:       # selective recompute: keep only this sub-module's input, rebuild its internals in backward
            attn = torch.utils.checkpoint.checkpoint(self.self_attn, normed, ctx, None, use_reentrant=False)
        else:
            attn = self.self_attn(normed, ctx, cache)
        if self.residual_multiplier != 1.0:      # the residual add happens inside the next norm: scale the branch first
            attn = attn * self.residual_multiplier
        normed, residual = self.post_attention_layernorm(attn, residual)
        out = torch.utils.checkpoint.checkpoint(self.mlp, normed, use_reentrant=False) if "mlp" in sel else self.mlp(normed)
        if self.residual_multiplier != 1.0:
            out = out * self.residual_multiplier
        return out, residual


class MTPLayer(nn.Module):
    """Multi-token prediction block: h' = eh_proj([enorm(emb(tokens shifted by depth)); hnorm(h)]) -> decoder layer
    (paddleformers/transformers/deepseek_v3/modeling.py:1032-1128)."""

    def __init__(self, config: DecoderConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        # under sequence parallelism the layer works on this rank's token slice: its replicated weights collect partial
        # gradients, which are summed over the group before the optimizer step
        sp = bool(getattr(config, "sequence_parallel", False)) and get_parallel_state().degrees.mp > 1
        self.enorm = RMSNorm(config.hidden_size, config.rms_norm_eps, sp, dtype=dtype, device=device)
        self.hnorm = RMSNorm(config.hidden_size, config.rms_norm_eps, sp, dtype=dtype, device=device)
        self.eh_proj = nn.Linear(2 * config.hidden_size, config.hidden_size, bias=False, dtype=dtype, device=device)
        if sp:
            mark_as_sequence_parallel_parameter(self.eh_proj.weight)
        self.block = DecoderLayer(config, layer_idx, dtype=dtype, device=device)
        self.final_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps, sp, dtype=dtype, device=device)

    def forward(self, h2d, shifted_emb2d, ctx):
        x = torch.cat([self.enorm(shifted_emb2d), self.hnorm(h2d)], dim=-1)
        x = _apply(self.eh_proj, x)
        out, res = self.block(x, None, ctx)
        return self.final_layernorm(out, res)[0]


class DecoderModel(nn.Module):
    def __init__(self, config: DecoderConfig, dtype=None, device=None, layer_range: Optional[range] = None,
                 with_embedding: bool = True, with_final_norm: bool = True):
        super().__init__()
        ps = get_parallel_state()
        self.config = config
        self.sp = bool(getattr(config, "sequence_parallel", False)) and ps.degrees.mp > 1
        self.layer_range = layer_range if layer_range is not None else range(config.num_hidden_layers)
        if with_embedding:
            if ps.degrees.mp > 1:
                self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size, self.sp, dtype=dtype, device=device)
            else:
                self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, dtype=dtype, device=device)
        else:
            self.embed_tokens = None
        self.layers = nn.ModuleDict({str(i): DecoderLayer(config, i, dtype=dtype, device=device) for i in self.layer_range})
        self.norm = make_norm(config, config.hidden_size, self.sp, dtype=dtype, device=device) if with_final_norm else None
        self._rope_cache = {}

    # ------------------------------------------------------------------ helpers
    def rope(self, device, length: int, local: bool = False):
        """(cos, sin) tables; ``local``: the tables of sliding-window layers with their own base and no scaling rule."""
        cfg = self.config
        rot = int((cfg.qk_rope_head_dim if cfg.is_mla else cfg.head_dim * cfg.partial_rotary_factor))
        n = max(length, 1)
        kind = (cfg.rope_scaling or {}).get("rope_type", (cfg.rope_scaling or {}).get("type")) if not local else None
        # rules that depend on the sequence length get one table per regime (longrope: short / long factors) or per length
        # (dynamic NTK beyond the trained context)
        regime = F.rope_uses_long_factors(cfg.rope_scaling, n) if kind in ("longrope", "su") else \
            (n if kind == "dynamic" and n > cfg.max_position_embeddings else 0)
        key = (str(device), rot, local, regime)
        cached = self._rope_cache.get(key)
        if cached is None or cached[0].shape[0] < n:
            seq = n
            n = max(n, min(cfg.max_position_embeddings, 8192)) if kind != "dynamic" else n
            if local:
                cached = F.rope_tables(n, rot, float(cfg.rope_local_theta), device, None)
            else:
                cached = F.rope_tables(n, rot, cfg.rope_theta, device, cfg.rope_scaling, seq_len=seq,
                                       max_position_embeddings=cfg.max_position_embeddings)
            self._rope_cache[key] = cached
        return cached

    def make_context(self, input_ids, position_ids=None, kend=None, cp_positions=None, full_seq_len=None,
                     kend_full=None) -> BatchContext:
        B, S = input_ids.shape
        window = int(getattr(self.config, "sliding_window", None) or 0)
        if not any(self.config.layer_window(i) for i in self.layer_range):
            window = 0
        chunk = max([self.config.layer_chunk(i) for i in self.layer_range] or [0])
        kend_window = None
        if chunk and (full_seq_len or S) > chunk:
            if full_seq_len and full_seq_len != S:
                raise NotImplementedError("chunked attention is not combined with context / segment parallelism")
            # chunked layers: key j is visible up to the end of its own chunk (the same bound as a packed document of that length)
            j = torch.arange(S, device=input_ids.device, dtype=torch.int32)
            kend_window = ((j // chunk + 1) * chunk).clamp(max=S)[None].expand(B, S)
            if kend is not None:
                kend_window = torch.minimum(kend_window, kend.to(torch.int32).reshape(B, S))
            kend_window = kend_window.contiguous()
        elif window and (full_seq_len or S) > window:
            if full_seq_len and full_seq_len != S:
                raise NotImplementedError("sliding-window attention is not combined with context / segment parallelism")
            # key j stops being visible at row j + window; together with the causal rule this is the sliding window, and it
            # composes with document bounds by taking the smaller of the two
            kend_window = (torch.arange(S, device=input_ids.device, dtype=torch.int32) + window).clamp(max=S)[None].expand(B, S)
            if kend is not None:
                kend_window = torch.minimum(kend_window, kend.to(torch.int32).reshape(B, S))
            kend_window = kend_window.contiguous()
        max_pos = S if position_ids is None else max(S, int(self.config.max_position_embeddings))
        cos, sin = self.rope(input_ids.device, max_pos)
        pos = None
        if position_ids is not None:
            pos = position_ids.reshape(-1)
        elif B > 1:
            pos = torch.arange(S, device=input_ids.device).repeat(B)
        ps = get_parallel_state()
        S_full = 0
        if ps.degrees.cp > 1 and cp_positions is not None:
            S_full = int(full_seq_len or S * ps.degrees.cp)
        elif ps.degrees.sep > 1:
            S_full = int(full_seq_len or S * ps.degrees.sep)
        if S_full:
            cos, sin = self.rope(input_ids.device, max(max_pos, S_full))
        cos_l = sin_l = None
        if getattr(self.config, "rope_local_theta", None):
            cos_l, sin_l = self.rope(input_ids.device, max(max_pos, S_full), local=True)
        return BatchContext(B, S, pos, kend, cos, sin, cp_positions if S_full else None, S_full, kend_full if S_full else None,
                            kend_window, window, cos_l, sin_l)

    def token_slice(self, h):
        """This rank's rows of whole-sequence embeddings under sequence parallelism (the backward pass gathers the slices'
        gradients, so whatever produced the rows sees the gradient of all of them)."""
        return ScatterOp.apply(h, get_parallel_state().group("mp")) if self.sp else h

    def embed(self, input_ids, whole: bool = False):
        """[tokens, hidden] embeddings: this rank's token slice under sequence parallelism unless ``whole`` (multimodal models
        write feature rows over placeholder positions first and call ``token_slice`` afterwards)."""
        mult = float(getattr(self.config, "embedding_multiplier", 1.0) or 1.0)
        if isinstance(self.embed_tokens, VocabParallelEmbedding):
            h = self.embed_tokens(input_ids, whole=whole)
            h = h if h.dim() == 2 else h.reshape(-1, h.shape[-1])
        else:
            h = F.embedding(input_ids, self.embed_tokens.weight).reshape(-1, self.config.hidden_size)
        return h * mult if mult != 1.0 else h

    def run_layers(self, hidden, residual, ctx, caches=None):
        cfg = self.config
        recompute = self.training and getattr(cfg, "recompute_granularity", None) == "full"
        skip = set(getattr(cfg, "no_recompute_layers", None) or [])
        # recompute_method: "uniform" recomputes every layer (in chunks of recompute_num_layers, one checkpoint each);
        # "block" recomputes only the first recompute_num_layers layers of this stage and keeps the rest
        method = getattr(cfg, "recompute_method", None) or "uniform"
        n_rc = int(getattr(cfg, "recompute_num_layers", 1) or 1)
        layer_ids = list(self.layer_range)
        # refined_recompute = {operation: layers that recompute it}: the named operations of the other layers keep their saved
        # tensors and are skipped when the layer is rebuilt (utils/refined_recompute.py)
        refined = getattr(cfg, "refined_recompute", None) if recompute else None
        if refined:
            assert not getattr(cfg, "recompute_use_reentrant", False), "refined_recompute needs the non-reentrant checkpoint"
            assert not (method == "uniform" and n_rc > 1), "refined_recompute works per layer (recompute_num_layers 1)"
        if recompute and method == "block":
            skip |= set(layer_ids[n_rc:])
        if recompute and method == "uniform" and n_rc > 1 and caches is None:
            for j in range(0, len(layer_ids), n_rc):
                chunk = [self.layers[str(i)] for i in layer_ids[j:j + n_rc]]

                def run_chunk(h, r, chunk=chunk):
                    for lyr in chunk:
                        h, r = lyr(h, r, ctx, None)
                    return h, r

                hidden, residual = torch.utils.checkpoint.checkpoint(
                    run_chunk, hidden, residual, use_reentrant=bool(getattr(cfg, "recompute_use_reentrant", False)))
            return hidden, residual
        for i in self.layer_range:
            layer = self.layers[str(i)]
            cache = caches[i] if caches is not None else None
            if recompute and i not in skip and cache is None:
                kept = kept_ops_of_layer(refined, i, cfg.num_hidden_layers, layer_ids) if refined else ()
                if kept:
                    hidden, residual = checkpoint_keeping(lambda h, r, layer=layer: layer(h, r, ctx, None), kept, hidden, residual)
                    continue
                hidden, residual = torch.utils.checkpoint.checkpoint(
                    layer, hidden, residual, ctx, None, use_reentrant=bool(getattr(cfg, "recompute_use_reentrant", False)))
            else:
                hidden, residual = layer(hidden, residual, ctx, cache)
        return hidden, residual

    def forward(self, input_ids, position_ids=None, kend=None, caches=None, ctx: Optional[BatchContext] = None,
                cp_positions=None, full_seq_len=None, kend_full=None):
        ctx = ctx or self.make_context(input_ids, position_ids, kend, cp_positions, full_seq_len, kend_full)
        if getattr(self.config, "moe_router_load_balancing_type", "aux_loss") == "seq_aux_loss":
            for layer in self.layers.values():       # per-sequence balance loss: the router needs the rows-per-sequence of this batch
                gate = getattr(getattr(layer, "mlp", None), "gate", None)
                if gate is not None:
                    gate.tokens_per_seq = 0 if self.sp else ctx.S
        h = self.embed(input_ids)
        hidden, residual = self.run_layers(h, None, ctx, caches)
        if self.norm is not None:
            hidden = self.norm(hidden, residual)[0] if residual is not None else self.norm(hidden)
        return hidden, ctx


def label_norm(count):
    """Number of labelled tokens the loss is divided by. Ranks of a context / segment parallel group hold slices of ONE
    sequence: they normalise by the labelled tokens of the whole sequence (their mean per rank), so that averaging the
    ranks' losses and gradients gives the loss of the unsplit sequence even when labels are spread unevenly."""
    norm = count.clamp(min=1).to(torch.float32)
    ps = get_parallel_state()
    for axis in ("cp", "sep"):
        n_slices = getattr(ps.degrees, axis)
        if n_slices > 1 and torch.distributed.is_initialized():
            total = count.to(torch.float32)
            torch.distributed.all_reduce(total, group=ps.group(axis))
            norm = (total / n_slices).clamp(min=1.0)
    return norm


class DecoderForCausalLM(PretrainedModel, GenerationMixin):
    config_class = DecoderConfig
    base_model_prefix = "model"

    def __init__(self, config: DecoderConfig, dtype=None, device=None):
        super().__init__(config)
        dtype = dtype if dtype is not None else _resolve_dtype(config.dtype)
        ps = get_parallel_state()
        self.tp = ps.degrees.mp
        self.model = DecoderModel(config, dtype=dtype, device=device)
        self.sp = self.model.sp
        if config.tie_word_embeddings:
            self.lm_head = None
        elif self.tp > 1:
            self.lm_head = ColumnParallelLinear(config.hidden_size, config.vocab_size, bias=False,
                                                sequence_parallel=self.sp, dtype=dtype, device=device)
        else:
            self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False, dtype=dtype, device=device)
        n_mtp = int(getattr(config, "num_nextn_predict_layers", 0) or 0)
        self.mtp_layers = nn.ModuleList([MTPLayer(config, config.num_hidden_layers + i, dtype=dtype, device=device)
                                         for i in range(n_mtp)])
        self.ignore_index = -100
        self.loss_accumulation_steps = 1   # set by the trainer: folded into the in-forward loss scale
        self.post_init()

    # ------------------------------------------------------------------ weights
    def head_weight(self):
        return self.model.embed_tokens.weight if self.lm_head is None else self.lm_head.weight

    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, (nn.Linear, ColumnParallelLinear, RowParallelLinear)):
            nn.init.normal_(module.weight, 0.0, std)
            if getattr(module, "bias", None) is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, (nn.Embedding, VocabParallelEmbedding)):
            nn.init.normal_(module.weight, 0.0, std)
        elif isinstance(module, RMSNorm):
            nn.init.ones_(module.weight)
        else:
            from ..nn.moe import GroupedExperts, TopkRouter

            if isinstance(module, GroupedExperts):
                nn.init.normal_(module.gate_up_proj, 0.0, std)
                nn.init.normal_(module.down_proj, 0.0, std)
            elif isinstance(module, TopkRouter):
                nn.init.normal_(module.weight, 0.0, std)

    # ------------------------------------------------------------------ forward
    def compute_logits(self, hidden2d):
        w = self.head_weight()
        if self.tp > 1 and self.lm_head is not None:
            logits = self.lm_head(hidden2d)
        else:
            logits = F.linear(hidden2d, w)
        cap = float(getattr(self.config, "final_logit_softcapping", None) or 0.0)
        if cap:
            logits = (torch.tanh(logits.float() / cap) * cap).to(logits.dtype)
        return logits

    def full_logits(self, hidden2d):
        """[tokens, vocabulary] logits on every rank, differentiable. ``hidden2d`` is this rank's token slice under sequence
        parallelism, all tokens otherwise. Under tensor parallelism the head (or a tied vocabulary-parallel embedding) is a
        vocabulary shard: the hidden states are gathered / copied with a backward pass that sums the shards' gradients, the
        logit shards are concatenated with a backward pass that keeps this rank's shard."""
        if self.tp == 1:
            return self.compute_logits(hidden2d)
        group = get_parallel_state().group("mp")
        w = self.head_weight()
        h = AllGatherOp.apply(hidden2d, group) if self.sp else CopyToTP.apply(hidden2d, group)
        logits = F.linear(h, w)
        if w.shape[0] != self.config.vocab_size:
            logits = GatherLastDimOp.apply(logits, group)
        cap = float(getattr(self.config, "final_logit_softcapping", None) or 0.0)
        if cap:
            logits = (torch.tanh(logits.float() / cap) * cap).to(logits.dtype)
        return logits

    def _label_norm(self, count):
        return label_norm(count)

    def _filter_labelled_rows(self, hidden2d, labels_flat):
        """use_filtered_label_loss: only the rows whose label is not ignored go through the head GEMM and the loss (a large
        saving for SFT, where prompt tokens carry no label). Under sequence parallelism every rank filters its own token
        slice and the survivors are all-gathered with their varying counts. The row count depends on the data, so this
        reads it on the host (paddleformers/nn/criterion/sft_loss.py:138-157)."""
        keep = labels_flat != self.ignore_index
        if self.sp:
            from ..parallel.tensor_parallel import AllGatherVarlenOp

            g = get_parallel_state().group("mp")
            per = hidden2d.shape[0]
            r = torch.distributed.get_rank(g)
            local = keep[r * per:(r + 1) * per]
            rows = AllGatherVarlenOp.apply(hidden2d[local.nonzero(as_tuple=True)[0]], g)
        else:
            rows = hidden2d[keep.nonzero(as_tuple=True)[0]]
        return rows, labels_flat[keep]

    def _loss(self, hidden2d, labels_flat, scale, tokens_complete: bool = False):
        """(scaled loss sum, token count) of the head + cross entropy on hidden states [T, H]."""
        if getattr(self.config, "final_logit_softcapping", None):
            # capped logits cannot go through the fused head + loss kernel: head GEMM, cap and cross entropy run as separate
            # operations, in token chunks so that only a slice of the [tokens, vocabulary] logits is alive at a time
            assert self.tp == 1, "final logit soft-capping is implemented for tensor-parallel degree 1"
            total = hidden2d.new_zeros((), dtype=torch.float32)
            for lo in range(0, hidden2d.shape[0], 2048):
                lg = self.compute_logits(hidden2d[lo:lo + 2048]).float()
                total = total + torch.nn.functional.cross_entropy(lg, labels_flat[lo:lo + 2048], ignore_index=self.ignore_index,
                                                                  reduction="sum")
            return total * scale, (labels_flat != self.ignore_index).sum()
        if self.tp > 1:
            from ..parallel.vocab_parallel_loss import vocab_parallel_linear_cross_entropy

            h = hidden2d
            if self.sp and not tokens_complete:
                h = GatherOp.apply(h, get_parallel_state().group("mp"))
            return vocab_parallel_linear_cross_entropy(h, self.head_weight(), labels_flat, self.ignore_index, scale)
        chunk = int(getattr(self.config, "loss_subbatch_sequence_length", -1) or -1)
        return F.fused_linear_cross_entropy(hidden2d, self.head_weight(), labels_flat, self.ignore_index,
                                            chunk if chunk > 0 else 2048, scale)

    def forward(self, input_ids, labels=None, position_ids=None, attn_mask_startend_row_indices=None, kend=None,
                caches=None, return_logits: Optional[bool] = None, cp_global_positions=None, cp_full_seq_len=None,
                full_attn_mask_startend_row_indices=None, full_input_ids=None, full_labels=None, mtp_global_positions=None,
                **unused):
        """``labels`` are next-token targets aligned with ``input_ids`` (already shifted by the data pipeline, as in
        the reference's collators). ``attn_mask_startend_row_indices`` / ``kend``: int [B, S] FlashMask start rows.
        ``full_input_ids`` / ``full_labels`` / ``mtp_global_positions``: under context / segment parallelism the unsliced rows
        and the global position of every local token, for the multi-token-prediction heads."""
        if kend is None and attn_mask_startend_row_indices is not None:
            kend = attn_mask_startend_row_indices.reshape(input_ids.shape[0], -1)
        kend_full = full_attn_mask_startend_row_indices
        if kend_full is not None:
            kend_full = kend_full.reshape(input_ids.shape[0], -1)
        hidden, ctx = self.model(input_ids, position_ids, kend, caches, None, cp_global_positions, cp_full_seq_len, kend_full)
        logits_scaling = float(getattr(self.config, "logits_scaling", 1.0) or 1.0)
        if logits_scaling != 1.0:        # logits / s == head(hidden / s)
            hidden = hidden / logits_scaling
        out = CausalLMOutput()
        want_logits = return_logits if return_logits is not None else labels is None
        if want_logits:
            out.logits = self.full_logits(hidden).view(ctx.B, ctx.S, -1)
        if labels is not None:
            lab = labels.reshape(-1)
            count = (lab != self.ignore_index).sum()
            norm = self._label_norm(count)
            scale = 1.0 / (norm * float(self.loss_accumulation_steps))
            if getattr(self.config, "use_filtered_label_loss", False):
                rows, lab_kept = self._filter_labelled_rows(hidden, lab)
                loss, _ = self._loss(rows, lab_kept, scale, tokens_complete=True)
            else:
                loss, _ = self._loss(hidden, lab, scale)
            out.num_tokens = count
            if len(self.mtp_layers) > 0:
                # The fused head + loss functions write the head's weight gradient (already multiplied by their ``scale``)
                # into main_grad during the forward pass, so a factor applied to their result afterwards would reach dh but
                # not dW: the weight of the multi-token-prediction term, lam / depth, goes into the scale instead.
                lam = float(getattr(self.config, "mtp_loss_scaling_factor", 0.1))
                w = lam / len(self.mtp_layers)
                weighted = self._mtp_losses(hidden, input_ids, labels, ctx, scale, weight=w,
                                            full=(full_input_ids, full_labels, mtp_global_positions))
                out.mtp_losses = [l.detach() / w for l in weighted]
                loss = loss + torch.stack(weighted).sum()
            aux = [m.mlp.last_aux_loss for m in self.model.layers.values() if isinstance(m.mlp, MoELayer) and m.mlp.last_aux_loss is not None]
            if aux:
                out.aux_loss = torch.stack(aux).sum()
            out.loss = loss
        return out

    def _mtp_losses(self, hidden, input_ids, labels, ctx, scale, weight: float = 1.0, full=(None, None, None)):
        """Depth-k MTP head predicts token t+1+k from h_t and the embedding of token t+k; sequences are shifted left
        and the tail positions are ignored (paddleformers/nn/criterion/sft_loss.py:188-247). Every loss comes back already
        multiplied by ``weight``."""
        losses = []
        h = hidden                       # under sequence parallelism: this rank's token slice, like every layer input
        ids, lab = input_ids, labels
        full_ids, full_lab, gpos = full
        for k, layer in enumerate(self.mtp_layers, start=1):
            if full_ids is not None and gpos is not None:
                # this rank holds a slice of the sequence: token t + k and its label may live on another rank
                ahead = gpos + k
                inside = ahead < full_ids.shape[1]
                ahead = ahead.clamp(max=full_ids.shape[1] - 1)
                ids = full_ids.index_select(1, ahead)
                lab = torch.where(inside[None], full_lab.index_select(1, ahead), torch.full_like(lab, self.ignore_index))
            else:
                ids = torch.cat([ids[:, 1:], ids[:, -1:]], dim=1)
                lab = torch.cat([lab[:, 1:], torch.full_like(lab[:, -1:], self.ignore_index)], dim=1)
            if isinstance(self.model.embed_tokens, VocabParallelEmbedding):
                emb = self.model.embed_tokens(ids)          # token slices under sequence parallelism, whole rows otherwise
                emb = emb.reshape(-1, emb.shape[-1])
            else:
                emb = F.embedding(ids, self.model.embed_tokens.weight).reshape(-1, self.config.hidden_size)
            h = layer(h, emb, ctx)
            flat = lab.reshape(-1)
            cnt = (flat != self.ignore_index).sum()
            sc = weight / (self._label_norm(cnt) * float(self.loss_accumulation_steps))
            l, _ = self._loss(h, flat, sc)                  # gathers the token slices itself under sequence parallelism
            losses.append(l)
        return losses

    # ------------------------------------------------------------------ checkpoint mapping
    def weight_map(self) -> WeightMap:
        return build_weight_map(self.config)

    def get_hardware_flops_per_token(self, seq_len: int) -> float:
        from ..utils.flops import model_flops_per_token

        return model_flops_per_token(self.config, seq_len)


def _full_tokens(x, sp):
    if sp:
        return GatherOp.apply(x.reshape(-1, x.shape[-1]), get_parallel_state().group("mp"))
    return x.reshape(-1, x.shape[-1])


def _resolve_dtype(name):
    if isinstance(name, torch.dtype):
        return name
    return {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
            "float16": torch.float16, "fp16": torch.float16}.get(str(name).replace("torch.", ""), torch.float32)


def build_weight_map(config: DecoderConfig) -> WeightMap:
    """HF names -> fused internal parameters."""
    L = "model.layers.{L}."
    rules: List[Rule] = []
    per_layer: List[Rule] = []
    qkv_sizes = None
    # checkpoints trained with interleaved rotary pairs: q and k rows (sources 0 and 1) are permuted per head on load
    rope_perm = None
    if getattr(config, "rope_interleaved_checkpoint", False):
        rot = int(config.head_dim * float(getattr(config, "partial_rotary_factor", 1.0) or 1.0))
        spec = config.head_dim if rot == config.head_dim else (config.head_dim, 0, rot)       # only the rotated rows are paired
        rope_perm = {0: spec, 1: spec}
    mla_q_name = mla_q_perm = mla_kv_perm = None
    if config.is_mla:
        # MLA projections keep their HF names. DeepSeek checkpoints store the rotary slice of every query head and of the
        # compressed kv projection with interleaved pairs (the published model code rotates (2i, 2i + 1)); the rows are
        # permuted to the half-split order of the rotary kernels on load and back on save
        # (paddleformers/transformers/deepseek_v3/modeling.py:229-233 does the same permutation on activations).
        if getattr(config, "rope_interleave", True):
            qd = config.qk_nope_head_dim + config.qk_rope_head_dim
            mla_q_name = "q_b_proj.weight" if config.q_lora_rank else "q_proj.weight"
            mla_q_perm = {0: (qd, config.qk_nope_head_dim, config.qk_rope_head_dim)}
            mla_kv_perm = {0: (config.kv_lora_rank + config.qk_rope_head_dim, config.kv_lora_rank, config.qk_rope_head_dim)}
            per_layer.append(Rule(L + "self_attn." + mla_q_name, [L + "self_attn." + mla_q_name], rope_deinterleave=mla_q_perm))
            per_layer.append(Rule(L + "self_attn.kv_a_proj_with_mqa.weight", [L + "self_attn.kv_a_proj_with_mqa.weight"],
                                  rope_deinterleave=mla_kv_perm))
    else:
        qkv_sizes = [config.num_attention_heads * config.head_dim, config.num_key_value_heads * config.head_dim,
                     config.num_key_value_heads * config.head_dim]
        if getattr(config, "attention_output_gate", False):
            pass                                        # q (with its gate rows), k and v stay separate parameters under the same names
        elif getattr(config, "hf_fused_qkv", False):      # the checkpoint already stores [q | k | v] rows in one matrix
            groups = None
            if getattr(config, "qkv_grouped_by_kv_head", False):
                groups = (config.num_key_value_heads, config.num_attention_heads // config.num_key_value_heads, config.head_dim)
            per_layer.append(Rule(L + "self_attn.qkv_proj.weight", [L + "self_attn.qkv_proj.weight"], qkv_groups=groups))
        else:
            per_layer.append(Rule(L + "self_attn.qkv_proj.weight", [L + "self_attn.q_proj.weight", L + "self_attn.k_proj.weight",
                                                                     L + "self_attn.v_proj.weight"], "concat", 0, sizes=qkv_sizes,
                                  rope_deinterleave=rope_perm))
        if config.attention_bias and not getattr(config, "hf_fused_qkv", False) and not getattr(config, "attention_output_gate", False):
            per_layer.append(Rule(L + "self_attn.qkv_proj.bias", [L + "self_attn.q_proj.bias", L + "self_attn.k_proj.bias",
                                                                   L + "self_attn.v_proj.bias"], "concat", 0, sizes=qkv_sizes,
                                  rope_deinterleave=rope_perm))
    if getattr(config, "hf_fused_gate_up", False):  # [gate; up] rows already stacked in the checkpoint
        dense_rule = Rule(L + "mlp.gate_up_proj.weight", [L + "mlp.gate_up_proj.weight"])
    else:
        dense_rule = Rule(L + "mlp.gate_up_proj.weight", [L + "mlp.gate_proj.weight", L + "mlp.up_proj.weight"], "concat", 0)
    off = float(getattr(config, "norm_weight_offset", 0.0) or 0.0)
    if off:                                         # checkpoints that store (w - offset) for every RMSNorm weight
        rules.append(Rule("model.norm.weight", ["model.norm.weight"], offset=off))
        norm_names = ["input_layernorm.weight", "post_attention_layernorm.weight"]
        if getattr(config, "block_style", "pre") == "sandwich":
            norm_names += ["pre_feedforward_layernorm.weight", "post_feedforward_layernorm.weight"]
        if config.use_qk_norm and not config.is_mla:
            norm_names += ["self_attn.q_norm.weight", "self_attn.k_norm.weight"]
        for nm in norm_names:
            per_layer.append(Rule(L + nm, [L + nm], offset=off))
    qk_names = getattr(config, "qk_norm_hf_names", None)
    if qk_names and config.use_qk_norm and not config.is_mla:
        per_layer.append(Rule(L + "self_attn.q_norm.weight", [L + "self_attn." + qk_names[0] + ".weight"], offset=off))
        per_layer.append(Rule(L + "self_attn.k_norm.weight", [L + "self_attn." + qk_names[1] + ".weight"], offset=off))
    dense_rules = [dense_rule]
    if config.mlp_bias and not getattr(config, "hf_fused_gate_up", False):
        dense_rules.append(Rule(L + "mlp.gate_up_proj.bias", [L + "mlp.gate_proj.bias", L + "mlp.up_proj.bias"], "concat", 0))
    n_total = config.num_hidden_layers + int(getattr(config, "num_nextn_predict_layers", 0) or 0)
    for i in range(config.num_hidden_layers):
        rules.extend(expand_layers(per_layer, [i]))
        if getattr(config, "linear_attention_kind", None) == "lightning" and config.layer_types[i] == "linear_attention":
            a, b = f"model.layers.{i}.linear_attn.", f"model.layers.{i}.self_attn."
            rules += [Rule(a + "qkv.weight", [b + "qkv_proj.weight"]), Rule(a + "gate.weight", [b + "output_gate.weight"]),
                      Rule(a + "out.weight", [b + "out_proj.weight"]), Rule(a + "norm.weight", [b + "norm.weight"])]
        if config.is_moe_layer(i):
            E = config.num_experts
            pre = f"model.layers.{i}.mlp."
            # checkpoint-side names: the block ("mlp" unless the family says otherwise, e.g. Mixtral's "block_sparse_moe") and
            # the three expert projections (gate, up, down)
            src = f"model.layers.{i}." + (getattr(config, "moe_block_hf_name", None) or "mlp") + "."
            g_n, u_n, d_n = getattr(config, "expert_proj_hf_names", None) or ("gate_proj", "up_proj", "down_proj")
            if getattr(config, "moe_modality_isolated", False):
                # a text and a vision expert group: the checkpoint numbers the experts consecutively (text 0 .. E-1, vision
                # E .. 2E-1), stores both routers transposed ([H, E]; the vision one as "weight_1") and both correction biases
                # as the two rows of one tensor
                tr = (lambda t: t.t().contiguous(), lambda t: t.t().contiguous())
                for g, (part, wname) in enumerate((("text_moe.", "gate.weight"), ("vision_moe.", "gate.weight_1"))):
                    rules.append(Rule(pre + part + "experts.gate_up_proj", [src + "experts.{E}." + g_n + ".weight", src + "experts.{E}." + u_n + ".weight"],
                                      "stack_concat", 0, E, 2, expert_base=g * E))
                    rules.append(Rule(pre + part + "experts.down_proj", [src + "experts.{E}." + d_n + ".weight"], "stack", 0, E, expert_base=g * E))
                    rules.append(Rule(pre + part + "gate.weight", [src + wname], fn=tr))
                    if config.topk_method == "noaux_tc":
                        rules.append(Rule(pre + part + "gate.e_score_correction_bias", [src + "moe_statics.e_score_correction_bias"],
                                          fn=(lambda t, g=g: t[g], lambda t: t[None])))
                if config.n_shared_experts:
                    rules.append(Rule(pre + "shared_experts.gate_up_proj.weight",
                                      [src + "shared_experts.gate_proj.weight", src + "shared_experts.up_proj.weight"], "concat", 0))
                continue
            if getattr(config, "hf_experts_style", None) == "llama4":
                # stacked [E, H, 2I] ([in, out], gate columns then up columns) and [E, I, H]
                tr = (lambda t: t.transpose(1, 2).contiguous(), lambda t: t.transpose(1, 2).contiguous())
                rules.append(Rule(pre + "experts.gate_up_proj", [src + "experts.gate_up_proj"], fn=tr))
                rules.append(Rule(pre + "experts.down_proj", [src + "experts.down_proj"], fn=tr))
                rules.append(Rule(pre + "gate.weight", [src + config.router_weight_hf_name]))
                sh = config.shared_expert_hf_name
                rules.append(Rule(pre + "shared_experts.down_proj.weight", [src + sh + ".down_proj.weight"]))
                rules.append(Rule(pre + "shared_experts.gate_up_proj.weight", [src + sh + ".gate_proj.weight", src + sh + ".up_proj.weight"],
                                  "concat", 0))
                continue
            if getattr(config, "hf_experts_style", None) == "gpt_oss":
                # stacked [E, H, 2I] with gate / up columns interleaved, [E, I, H], and biases; router under "router"
                def split_cols(t):        # [..., 2I] interleaved -> [gate | up]
                    return torch.cat([t[..., 0::2], t[..., 1::2]], dim=-1)

                def join_cols(t):
                    g, u = t.chunk(2, dim=-1)
                    return torch.stack([g, u], dim=-1).flatten(-2)

                rules.append(Rule(pre + "experts.gate_up_proj", [src + "experts.gate_up_proj"],
                                  fn=(lambda t: split_cols(t).transpose(1, 2).contiguous(), lambda t: join_cols(t.transpose(1, 2)).contiguous())))
                rules.append(Rule(pre + "experts.gate_up_bias", [src + "experts.gate_up_proj_bias"], fn=(split_cols, join_cols)))
                rules.append(Rule(pre + "experts.down_proj", [src + "experts.down_proj"],
                                  fn=(lambda t: t.transpose(1, 2).contiguous(), lambda t: t.transpose(1, 2).contiguous())))
                rules.append(Rule(pre + "experts.down_bias", [src + "experts.down_proj_bias"]))
                rules.append(Rule(pre + "gate.weight", [src + "router.weight"]))
                rules.append(Rule(pre + "gate.bias", [src + "router.bias"]))
                continue
            if getattr(config, "hf_fused_experts", False):     # the checkpoint stores the stacked [E, 2I, H] / [E, H, I] tensors
                rules.append(Rule(pre + "experts.gate_up_proj", [src + "experts.gate_up_proj"]))
                rules.append(Rule(pre + "experts.down_proj", [src + "experts.down_proj"]))
            else:
                rules.append(Rule(pre + "experts.gate_up_proj", [src + "experts.{E}." + g_n + ".weight", src + "experts.{E}." + u_n + ".weight"],
                                  "stack_concat", 0, E, 2))
                rules.append(Rule(pre + "experts.down_proj", [src + "experts.{E}." + d_n + ".weight"], "stack", 0, E))
            if getattr(config, "router_weight_hf_name", None) or src != pre:
                rules.append(Rule(pre + "gate.weight", [src + (getattr(config, "router_weight_hf_name", None) or "gate.weight")]))
            if getattr(config, "router_bias_name", None) and config.topk_method == "noaux_tc":
                # stored outside the gate module (and, in some families, with a leading unit dimension)
                rules.append(Rule(pre + "gate.e_score_correction_bias", [f"model.layers.{i}." + config.router_bias_name],
                                  flatten=bool(getattr(config, "router_bias_leading_dim", True))))
            if config.n_shared_experts:
                sh = getattr(config, "shared_expert_hf_name", "shared_experts")
                if sh != "shared_experts" or src != pre:
                    rules.append(Rule(pre + "shared_experts.down_proj.weight", [src + sh + ".down_proj.weight"]))
                rules.append(Rule(pre + "shared_experts.gate_up_proj.weight",
                                  [src + sh + ".gate_proj.weight", src + sh + ".up_proj.weight"], "concat", 0))
        else:
            rules.extend(expand_layers(dense_rules, [i]))
    # MTP layers are stored by HF DeepSeek-V3 / GLM-4.5 as extra entries of model.layers
    for k in range(n_total - config.num_hidden_layers):
        i = config.num_hidden_layers + k
        src, dst = f"model.layers.{i}.", f"mtp_layers.{k}."
        for name in ("enorm.weight", "hnorm.weight", "eh_proj.weight"):
            rules.append(Rule(dst + name, [src + name]))
        rules.append(Rule(dst + "final_layernorm.weight", [src + "shared_head.norm.weight"]))
        blk = dst + "block."
        for name in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.o_proj.weight"):
            rules.append(Rule(blk + name, [src + name]))
        if config.is_mla:
            for name in ("q_a_proj.weight", "q_a_layernorm.weight", "q_b_proj.weight", "kv_a_proj_with_mqa.weight",
                         "kv_a_layernorm.weight", "kv_b_proj.weight"):
                perm = mla_q_perm if name == mla_q_name else mla_kv_perm if name == "kv_a_proj_with_mqa.weight" else None
                rules.append(Rule(blk + "self_attn." + name, [src + "self_attn." + name], rope_deinterleave=perm))
        else:
            rules.append(Rule(blk + "self_attn.qkv_proj.weight", [src + "self_attn.q_proj.weight", src + "self_attn.k_proj.weight",
                                                                 src + "self_attn.v_proj.weight"], "concat", 0, sizes=qkv_sizes))
            if config.attention_bias:
                rules.append(Rule(blk + "self_attn.qkv_proj.bias", [src + "self_attn.q_proj.bias", src + "self_attn.k_proj.bias",
                                                                   src + "self_attn.v_proj.bias"], "concat", 0, sizes=qkv_sizes))
            if config.use_qk_norm:
                rules.append(Rule(blk + "self_attn.q_norm.weight", [src + "self_attn.q_norm.weight"]))
                rules.append(Rule(blk + "self_attn.k_norm.weight", [src + "self_attn.k_norm.weight"]))
        if config.is_moe_layer(i) or config.num_experts > 0:
            E = config.num_experts
            rules.append(Rule(blk + "mlp.gate.weight", [src + "mlp.gate.weight"]))
            if config.topk_method == "noaux_tc":
                rules.append(Rule(blk + "mlp.gate.e_score_correction_bias", [src + "mlp.gate.e_score_correction_bias"]))
            rules.append(Rule(blk + "mlp.experts.gate_up_proj", [src + "mlp.experts.{E}.gate_proj.weight", src + "mlp.experts.{E}.up_proj.weight"],
                              "stack_concat", 0, E, 2))
            rules.append(Rule(blk + "mlp.experts.down_proj", [src + "mlp.experts.{E}.down_proj.weight"], "stack", 0, E))
            if config.n_shared_experts:
                rules.append(Rule(blk + "mlp.shared_experts.gate_up_proj.weight",
                                  [src + "mlp.shared_experts.gate_proj.weight", src + "mlp.shared_experts.up_proj.weight"], "concat", 0))
                rules.append(Rule(blk + "mlp.shared_experts.down_proj.weight", [src + "mlp.shared_experts.down_proj.weight"]))
        else:
            rules.append(Rule(blk + "mlp.gate_up_proj.weight", [src + "mlp.gate_proj.weight", src + "mlp.up_proj.weight"], "concat", 0))
            rules.append(Rule(blk + "mlp.down_proj.weight", [src + "mlp.down_proj.weight"]))
    translation = getattr(config, "hf_name_translation", None)
    if translation:
        # families that store the same tensors under other names: parameters that would keep their name get an explicit
        # rule, then every checkpoint-side name is rewritten
        have = {r.target for r in rules}
        same = ["model.embed_tokens.weight", "model.norm.weight"] + ([] if config.tie_word_embeddings else ["lm_head.weight"])
        for i in range(config.num_hidden_layers):
            pre = f"model.layers.{i}."
            same += [pre + "self_attn.o_proj.weight", pre + "input_layernorm.weight", pre + "post_attention_layernorm.weight"]
            if not config.is_moe_layer(i):
                same.append(pre + "mlp.down_proj.weight")
        rules += [Rule(n, [n]) for n in same if n not in have]

        def rewrite(name):
            for a, b in translation:
                name = name.replace(a, b)
            return name

        for r in rules:
            r.sources = [rewrite(x) for x in r.sources]
    return WeightMap(rules, translation)


def _family(name, cfg_cls):
    cls = type(name, (DecoderForCausalLM,), {"config_class": cfg_cls, "__doc__": f"{cfg_cls.model_type} causal LM (unified decoder)."})
    return cls


LlamaForCausalLM = _family("LlamaForCausalLM", LlamaConfig)
Qwen2ForCausalLM = _family("Qwen2ForCausalLM", Qwen2Config)
Qwen3ForCausalLM = _family("Qwen3ForCausalLM", Qwen3Config)
Qwen3MoeForCausalLM = _family("Qwen3MoeForCausalLM", Qwen3MoeConfig)
DeepseekV3ForCausalLM = _family("DeepseekV3ForCausalLM", DeepseekV3Config)
Glm4MoeForCausalLM = _family("Glm4MoeForCausalLM", Glm4MoeConfig)
MistralForCausalLM = _family("MistralForCausalLM", MistralConfig)
Phi3ForCausalLM = _family("Phi3ForCausalLM", Phi3Config)
SeedOssForCausalLM = _family("SeedOssForCausalLM", SeedOssConfig)
InternLM3ForCausalLM = _family("InternLM3ForCausalLM", InternLM3Config)
Ernie4_5ForCausalLM = _family("Ernie4_5ForCausalLM", Ernie4_5Config)
Ernie4_5MoeForCausalLM = _family("Ernie4_5MoeForCausalLM", Ernie4_5MoeConfig)
Qwen2MoeForCausalLM = _family("Qwen2MoeForCausalLM", Qwen2MoeConfig)
GraniteForCausalLM = _family("GraniteForCausalLM", GraniteConfig)
MiniCPMForCausalLM = _family("MiniCPMForCausalLM", MiniCPMConfig)
MiniCPM4_1ForCausalLM = _family("MiniCPM4_1ForCausalLM", MiniCPM4_1Config)
Glm4ForCausalLM = _family("Glm4ForCausalLM", Glm4Config)
Olmo2ForCausalLM = _family("Olmo2ForCausalLM", Olmo2Config)
GemmaForCausalLM = _family("GemmaForCausalLM", GemmaConfig)
Gemma2ForCausalLM = _family("Gemma2ForCausalLM", Gemma2Config)
Gemma3ForCausalLM = _family("Gemma3ForCausalLM", Gemma3TextConfig)
CohereForCausalLM = _family("CohereForCausalLM", CohereConfig)
Cohere2ForCausalLM = _family("Cohere2ForCausalLM", Cohere2Config)
StableLmForCausalLM = _family("StableLmForCausalLM", StableLmConfig)
HunYuanDenseV1ForCausalLM = _family("HunYuanDenseV1ForCausalLM", HunYuanDenseV1Config)
HunYuanMoEV1ForCausalLM = _family("HunYuanMoEV1ForCausalLM", HunYuanMoEV1Config)
MiniMaxM2ForCausalLM = _family("MiniMaxM2ForCausalLM", MiniMaxM2Config)
MiniMaxForCausalLM = _family("MiniMaxForCausalLM", MiniMaxConfig)
DiffLlamaForCausalLM = _family("DiffLlamaForCausalLM", DiffLlamaConfig)
MixtralForCausalLM = _family("MixtralForCausalLM", MixtralConfig)
MiniCPM3ForCausalLM = _family("MiniCPM3ForCausalLM", MiniCPM3Config)
InternLM2ForCausalLM = _family("InternLM2ForCausalLM", InternLM2Config)
GptOssForCausalLM = _family("GptOssForCausalLM", GptOssConfig)
Llama4ForCausalLM = _family("Llama4ForCausalLM", Llama4TextConfig)
Qwen3NextForCausalLM = _family("Qwen3NextForCausalLM", Qwen3NextConfig)
Qwen3_5ForCausalLM = _family("Qwen3_5ForCausalLM", Qwen3_5TextConfig)
Qwen3_5MoeForCausalLM = _family("Qwen3_5MoeForCausalLM", Qwen3_5MoeTextConfig)

class _ModelMapping(dict):
    """model_type -> causal-LM class; families that are models of their own are imported on first use."""

    def __missing__(self, key):
        from .configuration import STANDALONE_FAMILIES, _standalone

        if key not in STANDALONE_FAMILIES:
            raise KeyError(key)
        self[key] = _standalone(key, 1)
        return self[key]

    def __contains__(self, key):
        from .configuration import STANDALONE_FAMILIES

        return dict.__contains__(self, key) or key in STANDALONE_FAMILIES


MODEL_MAPPING = _ModelMapping({
    "llama": LlamaForCausalLM, "mistral": MistralForCausalLM, "phi3": Phi3ForCausalLM, "phi4": Phi3ForCausalLM, "phi4flash": Phi3ForCausalLM,
    "qwen2_moe": Qwen2MoeForCausalLM, "granite": GraniteForCausalLM, "minicpm": MiniCPMForCausalLM, "minicpm4_1": MiniCPM4_1ForCausalLM, "glm4": Glm4ForCausalLM, "olmo2": Olmo2ForCausalLM, "gemma": GemmaForCausalLM, "gemma2": Gemma2ForCausalLM, "gemma3_text": Gemma3ForCausalLM, "cohere": CohereForCausalLM, "cohere2": Cohere2ForCausalLM,
    "stablelm": StableLmForCausalLM, "hunyuan_v1_dense": HunYuanDenseV1ForCausalLM, "hunyuan_v1_moe": HunYuanMoEV1ForCausalLM, "minimax_m2": MiniMaxM2ForCausalLM, "minimax": MiniMaxForCausalLM, "diffllama": DiffLlamaForCausalLM, "mixtral": MixtralForCausalLM, "minicpm3": MiniCPM3ForCausalLM, "internlm2": InternLM2ForCausalLM, "gpt_oss": GptOssForCausalLM, "llama4_text": Llama4ForCausalLM, "qwen3_next": Qwen3NextForCausalLM, "qwen3_5_text": Qwen3_5ForCausalLM, "qwen3_5_moe_text": Qwen3_5MoeForCausalLM,
    "qwen3_5": Qwen3_5ForCausalLM, "qwen3_5_moe": Qwen3_5MoeForCausalLM,
    "glm_moe_dsa": DeepseekV3ForCausalLM, "deepseek_v32": DeepseekV3ForCausalLM, "kimi_k2": DeepseekV3ForCausalLM, "ernie4_5": Ernie4_5ForCausalLM, "ernie4_5_moe": Ernie4_5MoeForCausalLM, "seed_oss": SeedOssForCausalLM, "internlm3": InternLM3ForCausalLM, "glm4_moe_lite": DeepseekV3ForCausalLM, "qwen2": Qwen2ForCausalLM, "qwen3": Qwen3ForCausalLM,
    "qwen3_moe": Qwen3MoeForCausalLM, "deepseek_v3": DeepseekV3ForCausalLM, "deepseek_v2": DeepseekV3ForCausalLM,
    "glm4_moe": Glm4MoeForCausalLM, "decoder": DecoderForCausalLM,
})
