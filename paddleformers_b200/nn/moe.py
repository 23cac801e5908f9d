"""Mixture-of-experts building blocks: routers, token permutation, expert MLPs and the MoE layer.

Behaviour follows the reference's gates and layers:
* score functions in fp32, greedy / group-limited / ``noaux_tc`` top-k with a correction bias that only affects the
  selection, optional renormalisation and ``routed_scaling_factor``
  (paddleformers/nn/moe_deepep/moe_gate.py:31-52, :275-362; paddleformers/transformers/deepseek_v3/modeling.py:341;
  paddleformers/transformers/glm4_moe/modeling.py:333-385);
* the Switch/HF load-balancing auxiliary loss (paddleformers/transformers/qwen3_moe/modeling.py:1135) and z-loss
  (moe_gate.py:160-171), attached to the output with a pass-through autograd node
  (paddleformers/nn/moe_deepep/modular_moe_layer.py:267-269);
* stacked expert weights ``[E, 2I, H]`` / ``[E, H, I]`` (paddleformers/nn/experts.py:39-48), rows of every expert
  padded to a multiple of 128 so that a single grouped GEMM covers all local experts
  (paddleformers/cli/train/deepseek_v3_pretrain/moe_utils.py:143-262);
* an expert-usage counter that feeds the aux-loss-free bias update callback (moe_gate.py:446-451).
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from ..parallel.topology import get_parallel_state


class AddAuxiliaryLoss(torch.autograd.Function):
    """Returns ``x`` unchanged and injects d(aux)/d(...) = scale into the graph of ``aux`` during backward."""

    @staticmethod
    def forward(ctx, x, aux):
        ctx.save_for_backward(aux)
        return x

    @staticmethod
    def backward(ctx, g):
        (aux,) = ctx.saved_tensors
        return g, torch.ones_like(aux)


class _FusedRouteFn(torch.autograd.Function):
    """Scores, top-k, combine weights, per-expert counts, stable ranks and balance loss in two kernel launches
    (``csrc/moe_route.cu``); the backward pass recomputes the scores and returns d(logits) in one launch."""

    @staticmethod
    def forward(ctx, logits, sel_bias, k, sigmoid, n_group, topk_group, group_top2, norm_topk, scale, aux_coef, usage):
        T, E = logits.shape
        prob_sums = torch.zeros(E, dtype=torch.float32, device=logits.device) if aux_coef > 0 else None
        idx, w, rank, counts = torch.ops.pfb200.moe_route_fwd(logits, sel_bias, k, sigmoid, n_group, topk_group, group_top2,
                                                              norm_topk, scale, prob_sums, usage)
        aux = logits.new_zeros(())
        frac = None
        if aux_coef > 0:
            frac = counts.float() / max(T, 1)
            aux = aux_coef * E * (frac * (prob_sums / max(T, 1))).sum()
        ctx.save_for_backward(logits, idx, frac if frac is not None else logits.new_zeros(0))
        ctx.cfg = (sigmoid, norm_topk, scale, aux_coef, T, E)
        ctx.mark_non_differentiable(idx, rank, counts)
        return idx, w, aux, rank, counts

    @staticmethod
    def backward(ctx, d_idx, dw, daux, d_rank, d_counts):
        logits, idx, frac = ctx.saved_tensors
        sigmoid, norm_topk, scale, aux_coef, T, E = ctx.cfg
        aux_vec = None
        if aux_coef > 0 and daux is not None:
            aux_vec = (daux.float() * (aux_coef * E / max(T, 1))) * frac
        if dw is None:
            dw = torch.zeros(idx.shape, dtype=torch.float32, device=logits.device)
        dlogits = torch.ops.pfb200.moe_route_bwd(logits, None, idx, dw.float().contiguous(), aux_vec, sigmoid, norm_topk, scale)
        return (dlogits,) + (None,) * 10


def _global_balance_stats(frac: torch.Tensor, pmean: torch.Tensor):
    """Mean of the per-rank expert loads and mean routing probabilities over the data ranks; the result keeps the
    gradient of this rank's own probabilities (the other ranks' enter as constants)."""
    import torch.distributed as dist

    from ..parallel.topology import get_parallel_state

    ps = get_parallel_state()
    n = ps.size("dp_sharding_cp") if dist.is_initialized() else 1
    if n <= 1:
        return frac, pmean
    group = ps.group("dp_sharding_cp")
    both = torch.stack([frac.detach(), pmean.detach()])
    dist.all_reduce(both, group=group)
    return both[0] / n, (both[1] - pmean.detach() + pmean) / n


class _RandomLogits(torch.autograd.Function):
    """Standard-normal logits in the forward pass, the incoming gradient unchanged in the backward pass."""

    @staticmethod
    def forward(ctx, logits):
        return torch.randn_like(logits)

    @staticmethod
    def backward(ctx, g):
        return g


class TopkRouter(nn.Module):
    def _capacity_mask(self, idx: torch.Tensor, w: torch.Tensor, T: int, E: int) -> torch.Tensor:
        """1 for routed pairs inside their expert's capacity, 0 for dropped ones; no host synchronisation."""
        cap = int(math.ceil(self.capacity_factor * T * self.top_k / E))
        flat_e = idx.reshape(-1)
        n = flat_e.numel()
        if self.drop_policy == "position":
            prio = torch.arange(n, device=idx.device, dtype=torch.float32)              # earlier pairs first
        else:
            prio = -w.reshape(-1).float()                                               # larger probability first
        # rank of every pair inside its expert by priority: sort by (expert, priority)
        order = torch.argsort(prio, stable=True)
        order = order[torch.argsort(flat_e[order], stable=True)]
        counts = count_ids(flat_e, E)
        first = torch.cumsum(counts, 0) - counts
        rank_sorted = torch.arange(n, device=idx.device) - first[flat_e[order]]
        rank = torch.empty_like(rank_sorted)
        rank[order] = rank_sorted
        return (rank < cap).view_as(idx)

    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        self.num_experts = config.num_experts
        self.top_k = config.num_experts_per_tok
        self.scoring = config.scoring_func
        self.method = config.topk_method
        self.n_group = max(int(config.n_group or 1), 1)
        if self.method == "greedy":
            self.n_group = 1          # plain top-k ignores the expert groups (only the group-limited methods use them)
        self.topk_group = max(int(config.topk_group or 1), 1)
        self.norm_topk_prob = config.norm_topk_prob
        self.scale = float(config.routed_scaling_factor or 1.0)
        self.aux_coef = float(config.router_aux_loss_coef or 0.0)
        self.z_coef = float(config.router_z_loss_coef or 0.0)
        self.force_balance = bool(getattr(config, "moe_router_force_load_balancing", False))
        # global_aux_loss: the balance term uses the expert load and mean probability of ALL data ranks (one small
        # all-reduce each), not of this rank's tokens only; the gradient flows through the local probabilities
        # (examples/experiments/ernie_pretrain/models/moe/top2_gate.py:61-72)
        self.global_aux = bool(getattr(config, "global_aux_loss", False))
        # "seq_aux_loss": the balance term is computed per sequence and averaged, which also balances experts inside every
        # sequence rather than only over the batch (paddleformers/nn/moe_deepep/moe_gate.py:126-158)
        self.balance_type = str(getattr(config, "moe_router_load_balancing_type", "aux_loss") or "aux_loss")
        self.tokens_per_seq = 0      # set by the decoder model when rows are laid out sequence after sequence
        # capacity: every expert serves at most ceil(factor * tokens * top_k / experts) routed pairs; the rest are dropped
        # (their combine weight becomes zero) by position in the batch or by routing probability
        # (paddleformers/nn/moe_deepep/moe_gate.py:75-97, :183-273)
        self.capacity_factor = float(getattr(config, "moe_capacity_factor", 0.0) or 0.0)
        self.drop_policy = str(getattr(config, "moe_drop_policy", "probs") or "probs")
        # the router runs in fp32 like the reference's gate (weights kept fp32 regardless of the model dtype)
        self.weight = nn.Parameter(torch.empty(self.num_experts, config.hidden_size, dtype=torch.float32, device=device))
        self.weight.keep_fp32 = True
        # gpt-oss: the router has a bias and the combine weights are a softmax over the k selected LOGITS
        self.bias = nn.Parameter(torch.zeros(self.num_experts, dtype=torch.float32, device=device)) \
            if getattr(config, "router_bias", False) else None
        if self.bias is not None:
            self.bias.keep_fp32 = True
        if self.method == "noaux_tc":
            self.register_buffer("e_score_correction_bias", torch.zeros(self.num_experts, dtype=torch.float32, device=device))
        else:
            self.e_score_correction_bias = None
        self.register_buffer("expert_usage", torch.zeros(self.num_experts, dtype=torch.int64, device=device), persistent=False)

    def _fused_ok(self, logits: torch.Tensor) -> bool:
        """The routing kernel covers softmax / sigmoid scores with plain, group-limited or bias-corrected top-k and the
        batch-level balance loss; capacity dropping, per-sequence balance, z-loss and the biased / logit-scored routers
        stay on the tensor-operation path below."""
        E = self.num_experts
        if not (logits.is_cuda and os.environ.get("PFB_FUSED_ROUTER", "1") != "0" and F.use_cuda_kernels(logits)
                and hasattr(torch.ops.pfb200, "moe_route_fwd")):
            return False
        if self.scoring not in ("softmax", "sigmoid") or self.bias is not None or self.capacity_factor > 0:
            return False
        if self.global_aux and self.training and self.aux_coef > 0:
            return False
        if self.z_coef > 0 or self.balance_type not in ("aux_loss", "none") or E % 32 != 0 or E > 256 or self.top_k > 32:
            return False
        if self.n_group > 1 and ((E // 32) % self.n_group != 0 or self.topk_group > self.n_group):
            return False
        return True

    def forward(self, x2d: torch.Tensor):
        """x2d: [T, H] -> (topk_idx [T,k] int64, topk_weight [T,k] fp32, aux_loss scalar or None)."""
        logits = F.router_logits(x2d, self.weight)
        self.last_plan = None
        if self._fused_ok(logits):
            if self.force_balance:
                # benchmarking with random-initialised weights: the experts are chosen from random logits so that every
                # expert gets its share of the tokens (a deep random network routes almost all tokens to a few experts);
                # the gate GEMM, the routing kernel and the work per token are unchanged
                logits = _RandomLogits.apply(logits)
            want_aux = self.training and self.aux_coef > 0 and self.balance_type != "none"
            idx, w, aux, rank, counts = _FusedRouteFn.apply(
                logits.contiguous(), self.e_score_correction_bias, self.top_k, self.scoring == "sigmoid", self.n_group,
                self.topk_group, self.method == "noaux_tc", bool(self.norm_topk_prob and self.top_k > 1), self.scale,
                self.aux_coef if want_aux else 0.0, self.expert_usage)
            # the dispatcher reuses the kernel's per-expert counts and stable ranks instead of sorting the pairs again
            self.last_plan = {"idx": idx, "rank_in_expert": rank, "counts": counts}
            return idx, w, (aux if want_aux else None)
        if self.bias is not None:
            logits = logits + self.bias
        if self.scoring == "sigmoid_topk_logits":        # Llama 4: experts by logit, weight = sigmoid of the selected logit
            top, idx = logits.topk(self.top_k, dim=-1)
            with torch.no_grad():
                self.expert_usage.scatter_add_(0, idx.reshape(-1), torch.ones_like(idx.reshape(-1)))
            return idx, torch.sigmoid(top) * self.scale, None
        if self.scoring == "softmax_topk":
            top, idx = logits.topk(self.top_k, dim=-1)
            w = torch.softmax(top, dim=-1) * self.scale
            with torch.no_grad():
                self.expert_usage.scatter_add_(0, idx.reshape(-1), torch.ones_like(idx.reshape(-1)))
            aux = None
            if self.training and self.aux_coef > 0 and self.balance_type != "none":
                T, E = logits.shape
                probs = torch.softmax(logits, dim=-1)
                frac = torch.zeros(E, dtype=torch.float32, device=x2d.device).scatter_add_(
                    0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=x2d.device)) / max(T, 1)
                aux = self.aux_coef * E * (frac * probs.mean(0)).sum()
            return idx, w, aux
        if self.scoring == "sigmoid":
            scores = torch.sigmoid(logits)
        else:
            scores = torch.softmax(logits, dim=-1)
        T, E = scores.shape
        if self.force_balance:
            base = torch.arange(T, device=x2d.device)[:, None] * self.top_k + torch.arange(self.top_k, device=x2d.device)[None]
            idx = base % E
        else:
            sel = scores if self.e_score_correction_bias is None else scores + self.e_score_correction_bias[None]
            if self.n_group > 1:
                g = sel.view(T, self.n_group, E // self.n_group)
                if self.method == "noaux_tc":
                    gscore = g.topk(2, dim=-1)[0].sum(-1)
                else:
                    gscore = g.max(-1)[0]
                gidx = gscore.topk(self.topk_group, dim=-1)[1]
                gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1.0)
                sel = sel.masked_fill(~gmask[:, :, None].expand(-1, -1, E // self.n_group).reshape(T, E).bool(), float("-inf"))
            idx = sel.topk(self.top_k, dim=-1)[1]
        w = scores.gather(1, idx)
        if self.norm_topk_prob and self.top_k > 1:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        w = w * self.scale
        if self.capacity_factor > 0:
            w = w * self._capacity_mask(idx, w.detach(), T, E).to(w.dtype)
        with torch.no_grad():
            self.expert_usage.scatter_add_(0, idx.reshape(-1), torch.ones_like(idx.reshape(-1)))
        aux = None
        if self.training and (self.aux_coef > 0 or self.z_coef > 0):
            aux = x2d.new_zeros((), dtype=torch.float32)
            S = int(self.tokens_per_seq or 0)
            if self.aux_coef > 0 and self.balance_type == "seq_aux_loss" and 0 < S < T and T % S == 0:
                probs = scores if self.scoring == "softmax" else scores / (scores.sum(-1, keepdim=True) + 1e-20)
                nseq = T // S
                seq_of = (torch.arange(T, device=x2d.device) // S)[:, None].expand_as(idx)
                frac = torch.zeros(nseq * E, dtype=torch.float32, device=x2d.device).scatter_add_(
                    0, (seq_of * E + idx).reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=x2d.device))
                frac = frac.view(nseq, E) / S
                aux = aux + self.aux_coef * E * (frac * probs.view(nseq, S, E).mean(1)).sum(-1).mean()
            elif self.aux_coef > 0 and self.balance_type != "none":
                probs = scores if self.scoring == "softmax" else scores / (scores.sum(-1, keepdim=True) + 1e-20)
                frac = torch.zeros(E, dtype=torch.float32, device=x2d.device).scatter_add_(
                    0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=x2d.device)) / max(T, 1)
                pmean = probs.mean(0)
                if self.global_aux:
                    frac, pmean = _global_balance_stats(frac, pmean)
                aux = aux + self.aux_coef * E * (frac / self.top_k * pmean).sum() * self.top_k
            if self.z_coef > 0:
                aux = aux + self.z_coef * torch.logsumexp(logits, dim=-1).pow(2).mean()
        return idx, w, aux


# ---------------------------------------------------------------------------------------------------------------
# permutation into expert-sorted, 128-row padded segments
# ---------------------------------------------------------------------------------------------------------------
def count_ids(ids: torch.Tensor, n: int) -> torch.Tensor:
    """Histogram of ``ids`` (all in [0, n)) as int64 [n] without the host read-back that ``torch.bincount`` does."""
    return torch.zeros(n, dtype=torch.int64, device=ids.device).scatter_add_(0, ids, torch.ones_like(ids))


def build_dispatch_plan(idx: torch.Tensor, num_local_experts: int, expert_offset: int = 0, block: int = 128):
    """Sort (token, slot) pairs by expert and pad each expert segment to a multiple of ``block`` rows, entirely on
    the device (no host synchronisation: the padded buffer has a static upper-bound size).

    Returns (dest_row [T*k] int64 (-1 for pairs routed to non-local experts), block_expert [n_blocks] int32,
    padded_rows int (static upper bound), counts [E_local])."""
    T, k = idx.shape
    flat = idx.reshape(-1) - expert_offset
    local = (flat >= 0) & (flat < num_local_experts)
    e = torch.where(local, flat, torch.full_like(flat, num_local_experts))
    counts_all = count_ids(e, num_local_experts + 1)
    counts = counts_all[:num_local_experts]
    padded = (counts + block - 1) // block * block
    seg_start = torch.cumsum(padded, 0) - padded
    # rank of each pair inside its expert (stable): sort by expert, then position - first position of that expert
    order = torch.argsort(e, stable=True)
    sorted_e = e[order]
    first = torch.cumsum(counts_all, 0)
    first = torch.cat([first.new_zeros(1), first[:-1]])
    rank_sorted = torch.arange(e.numel(), device=e.device) - first[sorted_e]
    rank = torch.empty_like(rank_sorted)
    rank[order] = rank_sorted
    seg = torch.cat([seg_start, seg_start.new_zeros(1)])
    dest = torch.where(local, seg[e] + rank, torch.full_like(e, -1))
    max_rows = ((T * k + block - 1) // block + num_local_experts) * block
    n_blocks = max_rows // block
    # block -> expert table: block b belongs to expert j iff seg_start[j] <= b*block < seg_start[j] + padded[j]
    bpos = torch.arange(n_blocks, device=e.device) * block
    ends = seg_start + padded
    be = torch.searchsorted(ends, bpos, right=True)
    block_expert = torch.where(bpos < ends[-1] if num_local_experts > 0 else bpos < 0, be, torch.full_like(be, -1)).to(torch.int32)
    return dest, block_expert, max_rows, counts


class _PermuteFn(torch.autograd.Function):
    """rows[dest[p]] = x[p // k] for every routed pair p with dest >= 0 (padding rows stay zero)."""

    @staticmethod
    def forward(ctx, x, dest, k, rows):
        out = x.new_zeros((rows, x.shape[1]))
        valid = dest >= 0
        src_tok = torch.arange(dest.numel(), device=x.device) // k
        out.index_copy_(0, dest[valid], x[src_tok[valid]])
        ctx.save_for_backward(dest)
        ctx.k, ctx.T = k, x.shape[0]
        return out

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        valid = dest >= 0
        src_tok = torch.arange(dest.numel(), device=g.device) // ctx.k
        dx = g.new_zeros((ctx.T, g.shape[1]), dtype=torch.float32)
        dx.index_add_(0, src_tok[valid], g[dest[valid]].float())
        return dx.to(g.dtype), None, None, None


def unpermute_combine(y_rows: torch.Tensor, dest: torch.Tensor, weights: torch.Tensor, T: int) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * y_rows[dest[t*k + j]] (pairs with dest < 0 contribute nothing)."""
    k = weights.shape[1]
    valid = (dest >= 0)
    gathered = y_rows[dest.clamp(min=0)] * (weights.reshape(-1, 1) * valid[:, None]).to(y_rows.dtype)
    return gathered.view(T, k, -1).sum(1)


class GroupedExperts(nn.Module):
    """Stacked SwiGLU experts; local experts only (E_local = E / ep)."""

    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        ps = get_parallel_state()
        self.ep = ps.degrees.ep
        self.num_experts = config.num_experts
        assert self.num_experts % self.ep == 0
        self.num_local = self.num_experts // self.ep
        self.expert_offset = ps.rank_in("ep") * self.num_local if self.ep > 1 else 0
        H, I = config.hidden_size, config.moe_intermediate_size
        self.hidden, self.inter = H, I
        self.gate_up_proj = nn.Parameter(torch.empty(self.num_local, 2 * I, H, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(self.num_local, H, I, dtype=dtype, device=device))
        for p in (self.gate_up_proj, self.down_proj):
            p.is_expert = True           # gradients are reduced over the moe_sharding group only
            p.shard_spec = ("ep", 0, None)
        # config.fp8 = "e4m3": expert GEMMs of the forward and input-gradient passes run block-scaled fp8 on quantised
        # weight copies that are refreshed once per optimizer step; weight gradients stay in bf16
        self.use_fp8 = bool(getattr(config, "fp8", None)) and H % 128 == 0 and I % 128 == 0
        self._fp8_cache = None

    def refresh_fp8_weight_cache(self):
        """Quantise the expert weights (128x128 blocks) and their per-expert transposes for the input-gradient GEMMs
        (the cached ``fp8_weight`` / ``fp8_weight_transpose`` of paddleformers/transformers/fp8_utils.py:913-1009)."""
        if not (self.use_fp8 and self.gate_up_proj.is_cuda):
            self._fp8_cache = None
            return
        from ..quantization.fp8 import quant_weight_kernel

        E, N2, H = self.gate_up_proj.shape
        I = N2 // 2
        with torch.no_grad():
            gu, dn = self.gate_up_proj.detach(), self.down_proj.detach()
            c = {}
            c["gu_q"], c["gu_s"] = quant_weight_kernel(gu.reshape(E * N2, H))
            c["dn_q"], c["dn_s"] = quant_weight_kernel(dn.reshape(E * H, I))
            c["guT_q"], c["guT_s"] = quant_weight_kernel(gu.transpose(1, 2).contiguous().reshape(E * H, N2))
            c["dnT_q"], c["dnT_s"] = quant_weight_kernel(dn.transpose(1, 2).contiguous().reshape(E * I, H))
        self._fp8_cache = c

    def forward(self, rows: torch.Tensor, block_expert: torch.Tensor, counts: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, expert_rows: Optional[torch.Tensor] = None,
                grad_rows_out: Optional[torch.Tensor] = None):
        """rows: [R, H] expert-sorted with 128-row padded segments; returns [R, H] (written into ``out`` when given,
        e.g. a peer-visible buffer). ``expert_rows`` int32 [E, 2] = (first row, padded rows) per expert, if already
        known; ``grad_rows_out``: buffer that receives the gradient of ``rows`` in the backward pass. Rows of blocks
        that belong to no expert are left unwritten in every output."""
        if rows.is_cuda and rows.dtype == torch.bfloat16 and self.use_fp8:
            if self._fp8_cache is None:
                self.refresh_fp8_weight_cache()
            return _GroupedMlpFp8Fn.apply(rows, self.gate_up_proj, self.down_proj, block_expert, self._fp8_cache, out,
                                          expert_rows, grad_rows_out)
        if rows.is_cuda and rows.dtype == torch.bfloat16:
            return _GroupedMlpFn.apply(rows, self.gate_up_proj, self.down_proj, block_expert, out, expert_rows, grad_rows_out)
        out = torch.zeros_like(rows)
        be = block_expert.tolist()
        for b, e in enumerate(be):
            if e < 0:
                continue
            seg = rows[b * 128:(b + 1) * 128]
            gu = TF.linear(seg, self.gate_up_proj[e])
            g, u = gu.chunk(2, -1)
            out[b * 128:(b + 1) * 128] = TF.linear(TF.silu(g) * u, self.down_proj[e])
        return out


class BiasedGluExperts(GroupedExperts):
    """Experts with biases on both projections and gpt-oss's clamped gate: gate <= limit, |up| <= limit,
    out = (up + 1) * gate * sigmoid(alpha * gate). The grouped tcgen05 kernels fuse plain SwiGLU without biases, so these
    experts run block by block in tensor operations on every device: functional support, not a tuned path."""

    def __init__(self, config, dtype=None, device=None):
        super().__init__(config, dtype=dtype, device=device)
        self.gate_up_bias = nn.Parameter(torch.zeros(self.num_local, 2 * self.inter, dtype=dtype, device=device))
        self.down_bias = nn.Parameter(torch.zeros(self.num_local, self.hidden, dtype=dtype, device=device))
        for p in (self.gate_up_bias, self.down_bias):
            p.is_expert = True
            p.shard_spec = ("ep", 0, None)
        self.alpha = float(getattr(config, "glu_alpha", 1.702))
        self.limit = float(getattr(config, "swiglu_limit", 7.0))
        self.use_fp8 = False

    def forward(self, rows, block_expert, counts=None, out=None, expert_rows=None, grad_rows_out=None):
        if out is not None or grad_rows_out is not None:
            raise NotImplementedError("experts with biases take the all-to-all dispatcher (moe_token_dispatcher_type: alltoall)")
        pieces = []
        for b, e in enumerate(block_expert.tolist()):
            seg = rows[b * 128:(b + 1) * 128]
            if e < 0:
                pieces.append(torch.zeros_like(seg))
                continue
            gu = TF.linear(seg, self.gate_up_proj[e], self.gate_up_bias[e])
            g, u = gu.chunk(2, -1)
            g = g.clamp(max=self.limit)
            u = u.clamp(min=-self.limit, max=self.limit)
            pieces.append(TF.linear((u + 1) * g * torch.sigmoid(g * self.alpha), self.down_proj[e], self.down_bias[e]))
        return torch.cat(pieces, dim=0) if pieces else torch.zeros_like(rows)


class _GroupedMlpFn(torch.autograd.Function):
    """Two grouped tcgen05 GEMMs with the SwiGLU in the first epilogue. The backward runs grouped dgrad GEMMs and
    per-expert wgrad GEMMs accumulating into fp32 ``main_grad`` when present."""

    @staticmethod
    def forward(ctx, rows, w_gu, w_down, block_expert, out=None, expert_rows=None, grad_rows_out=None):
        E, N2, H = w_gu.shape
        I = N2 // 2
        R = rows.shape[0]
        # intermediate rows of unowned blocks are never read by the grouped kernels, so they need no initial value
        raw = torch.empty((R, N2), dtype=rows.dtype, device=rows.device)
        act = torch.empty((R, I), dtype=rows.dtype, device=rows.device)
        F.gemm(rows, w_gu.view(E * N2, H), out=act, epi=F.EPI_SWIGLU_BF16, out2=raw, block_expert=block_expert, n_per_expert=N2)
        if out is None:
            out = torch.zeros((R, H), dtype=rows.dtype, device=rows.device)
        else:
            ctx.mark_dirty(out)
        F.gemm(act, w_down.view(E * H, I), out=out, block_expert=block_expert, n_per_expert=H)
        ctx.save_for_backward(rows, w_gu, w_down, block_expert, raw)
        ctx.expert_rows = expert_rows
        ctx.grad_rows_out = grad_rows_out
        return out

    @staticmethod
    def backward(ctx, dout):
        rows, w_gu, w_down, block_expert, raw = ctx.saved_tensors
        E, N2, H = w_gu.shape
        I = N2 // 2
        R = rows.shape[0]
        dout = dout.contiguous()
        ops = torch.ops.pfb200
        # d(act) = dout @ W_down[e]  (grouped, B stored [H, I] per expert = MN-major for this product)
        dact = torch.empty((R, I), dtype=rows.dtype, device=rows.device)
        _grouped_dgrad(dout, w_down, dact, block_expert)
        dgu, act = ops.swiglu_bwd(dact, raw, True)
        drows = ctx.grad_rows_out if ctx.grad_rows_out is not None else torch.zeros((R, H), dtype=rows.dtype, device=rows.device)
        _grouped_dgrad(dgu, w_gu, drows, block_expert)
        # weight gradients: one wgrad GEMM per local expert over its row segment
        table = ctx.expert_rows if ctx.expert_rows is not None else expert_row_table(block_expert, E)
        dw_gu = _grouped_wgrad(dgu, rows, w_gu, table)
        dw_down = _grouped_wgrad(dout, act, w_down, table)
        return drows, dw_gu, dw_down, None, None, None, None


class _GroupedMlpFp8Fn(torch.autograd.Function):
    """Expert MLP with block-scaled e4m3 GEMMs: activations are quantised per 1x128 block on the fly, weights come from
    the per-step cache; the SwiGLU and the quantisation of its result are one kernel, and so are its backward and the
    quantisation of the gate / up gradients. Backward: input gradients through fp8 GEMMs on the
    transposed weight copies, weight gradients through the bf16 K-grouped kernel
    (paddleformers/transformers/fp8_utils.py:913-1190, FP8GroupGemmMlpFunctionNode)."""

    @staticmethod
    def forward(ctx, rows, w_gu, w_down, block_expert, cache, out=None, expert_rows=None, grad_rows_out=None):
        from ..quantization.fp8 import fp8_gemm, quant_act_kernel

        E, N2, H = w_gu.shape
        R = rows.shape[0]
        xq, xs_t = quant_act_kernel(rows)
        raw = torch.empty((R, N2), dtype=rows.dtype, device=rows.device)
        fp8_gemm(xq, xs_t, cache["gu_q"], cache["gu_s"], block_expert, N2, out=raw)
        aq, as_t, _ = torch.ops.pfb200.swiglu_quant_fwd(raw, None, True, False)    # SwiGLU and 1x128 quantisation in one pass
        if out is None:
            out = torch.zeros((R, H), dtype=rows.dtype, device=rows.device)
        else:
            ctx.mark_dirty(out)
        fp8_gemm(aq, as_t, cache["dn_q"], cache["dn_s"], block_expert, H, out=out)
        ctx.save_for_backward(rows, w_gu, w_down, block_expert, raw)
        ctx.cache, ctx.expert_rows, ctx.grad_rows_out = cache, expert_rows, grad_rows_out
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..quantization.fp8 import fp8_gemm, quant_act_kernel

        rows, w_gu, w_down, block_expert, raw = ctx.saved_tensors
        cache = ctx.cache
        E, N2, H = w_gu.shape
        I = N2 // 2
        R = rows.shape[0]
        dout = dout.contiguous()
        dq, ds_t = quant_act_kernel(dout)
        dact = torch.empty((R, I), dtype=rows.dtype, device=rows.device)
        fp8_gemm(dq, ds_t, cache["dnT_q"], cache["dnT_s"], block_expert, I, out=dact)
        dgu, gq, gs_t, act, _ = torch.ops.pfb200.swiglu_quant_bwd(dact, raw, None, True, True)
        drows = ctx.grad_rows_out if ctx.grad_rows_out is not None else torch.zeros((R, H), dtype=rows.dtype, device=rows.device)
        fp8_gemm(gq, gs_t, cache["guT_q"], cache["guT_s"], block_expert, H, out=drows)
        table = ctx.expert_rows if ctx.expert_rows is not None else expert_row_table(block_expert, E)
        dw_gu = _grouped_wgrad(dgu, rows, w_gu, table)
        dw_down = _grouped_wgrad(dout, act, w_down, table)
        return drows, dw_gu, dw_down, None, None, None, None, None


def _grouped_dgrad(dy, w, out, block_expert):
    """out[rows of e] = dy[rows of e] @ w[e], w: [E, N, K'] (contracts over N; the stacked weight is read MN-major,
    no transposed copy)."""
    E, N, Kp = w.shape
    F.gemm(dy, w.view(E * N, Kp), out=out, b_mn=True, block_expert=block_expert, n_per_expert=Kp)


def expert_row_table(block_expert: torch.Tensor, num_local: int) -> torch.Tensor:
    """int32 [E, 2] = (first row, row count) of each expert's padded segment, from the block -> expert table."""
    be = block_expert.to(torch.int64)
    cnt = count_ids(torch.where(be >= 0, be, torch.full_like(be, num_local)), num_local + 1)[:num_local] * 128
    start = torch.cumsum(cnt, 0) - cnt
    return torch.stack([start, cnt], dim=1).to(torch.int32).contiguous()


def _grouped_wgrad(dy, x, w, table):
    """dW[e] = dy[seg_e]^T @ x[seg_e] for all local experts in one launch (``table``: int32 [E, 2] row segments);
    accumulates into w.main_grad when present."""
    E, N, K = w.shape
    mg = getattr(w, "main_grad", None)
    target = mg.view(E, N, K) if mg is not None else torch.zeros((E, N, K), dtype=torch.float32, device=w.device)
    torch.ops.pfb200.gemm_wgrad_grouped(dy, x, target, table)
    return None if mg is not None else target.to(w.dtype)


class DenseMLP(nn.Module):
    """SwiGLU MLP with a fused gate|up projection (paddleformers/nn/mlp.py:113-130)."""

    def __init__(self, hidden_size: int, intermediate_size: int, config, bias: bool = False, tp: bool = True,
                 dtype=None, device=None):
        super().__init__()
        from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear

        sp = bool(getattr(config, "sequence_parallel", False)) and tp
        if tp and get_parallel_state().degrees.mp > 1:
            self.gate_up_proj = ColumnParallelLinear(hidden_size, 2 * intermediate_size, bias=bias,
                                                     sections=[intermediate_size, intermediate_size],
                                                     sequence_parallel=sp, epilogue="swiglu", dtype=dtype, device=device)
            self.down_proj = RowParallelLinear(intermediate_size, hidden_size, bias=bias, sequence_parallel=sp,
                                               dtype=dtype, device=device)
            self._tp = True
        else:
            self.gate_up_proj = nn.Linear(hidden_size, 2 * intermediate_size, bias=bias, dtype=dtype, device=device)
            self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=bias, dtype=dtype, device=device)
            self._tp = False
        # gate activation: "silu" runs in the fused SwiGLU kernels; the GELU variants (GeGLU families) use the unfused path
        self.act_name = str(getattr(config, "hidden_act", "silu") or "silu")
        if self.act_name not in ("silu", "swish"):
            assert not self._tp, "non-SiLU gated MLPs are implemented for tensor-parallel degree 1"

    def _gated_generic(self, x):
        gu = self.gate_up_proj(x) if not isinstance(self.gate_up_proj, nn.Linear) else \
            F.linear(x, self.gate_up_proj.weight, self.gate_up_proj.bias)
        g, u = gu.chunk(2, dim=-1)
        if self.act_name in ("gelu_pytorch_tanh", "gelu_tanh"):
            a = TF.gelu(g, approximate="tanh")
        elif self.act_name == "gelu":
            a = TF.gelu(g)
        else:
            a = getattr(TF, self.act_name)(g)
        dn = self.down_proj
        return F.linear(a * u, dn.weight, dn.bias) if isinstance(dn, nn.Linear) else dn(a * u)

    def forward(self, x):
        if self.act_name not in ("silu", "swish"):
            return self._gated_generic(x)
        from ..utils.refined_recompute import keep      # no-ops outside a refined-recompute frame

        if self._tp:
            return keep("mlp_row_ln", self.down_proj, keep("mlp_column_ln", self.gate_up_proj, x))
        gu, dn = self.gate_up_proj, self.down_proj
        if not isinstance(gu, nn.Linear):          # wrapped (e.g. LoRA): the wrapper owns the projection
            act = keep("mlp_column_ln", lambda t: F.swiglu(gu(t)), x)
        elif gu.bias is None:
            act = keep("mlp_column_ln", F.linear_swiglu, x, gu.weight)
        else:
            act = keep("mlp_column_ln", lambda t: F.swiglu(F.linear(t, gu.weight, gu.bias)), x)
        return keep("mlp_row_ln", F.linear, act, dn.weight, dn.bias) if isinstance(dn, nn.Linear) else keep("mlp_row_ln", dn, act)


class MoELayer(nn.Module):
    """Router -> dispatch (local permutation or expert-parallel exchange) -> grouped experts -> weighted combine,
    plus shared experts (paddleformers/nn/moe_deepep/modular_moe_layer.py:236-278)."""

    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        self.config = config
        self.gate = TopkRouter(config, dtype=dtype, device=device)
        experts_cls = BiasedGluExperts if getattr(config, "expert_bias", False) else GroupedExperts
        self.experts = experts_cls(config, dtype=dtype, device=device)
        self.shared_experts = None
        if config.n_shared_experts:
            si = config.shared_expert_intermediate_size or config.moe_intermediate_size * config.n_shared_experts
            self.shared_experts = DenseMLP(config.hidden_size, si, config, tp=False, dtype=dtype, device=device)
        # Qwen2-MoE: the shared expert's output is scaled per token by sigmoid(linear(x))
        self.shared_expert_gate = None
        if config.n_shared_experts and getattr(config, "shared_expert_gate", False):
            self.shared_expert_gate = nn.Linear(config.hidden_size, 1, bias=False, dtype=dtype, device=device)
        self.ep = get_parallel_state().degrees.ep
        self.last_aux_loss = None
        self._token_slices = 1
        if get_parallel_state().degrees.mp > 1 and getattr(config, "sequence_parallel", False):
            self._token_slices = get_parallel_state().degrees.mp
            # under sequence parallelism every tensor-parallel rank routes and computes ITS tokens with replicated router,
            # shared-expert and (without expert parallelism) expert weights: their gradients are partial sums over the
            # tokens and are added up over the group before the optimizer step
            # (paddleformers/trainer/trainer_callback.py:918-963 does this for the gate and the norm weights)
            from ..parallel.tensor_parallel import mark_as_sequence_parallel_parameter

            mods = [self.gate, self.shared_experts, self.shared_expert_gate] + ([self.experts] if self.ep == 1 else [])
            for mod in mods:
                for p in (mod.parameters() if mod is not None else ()):
                    mark_as_sequence_parallel_parameter(p)

    def forward(self, x2d: torch.Tensor) -> torch.Tensor:
        # moe_subbatch_token_num_before_dispatch > 0: route and run the experts on slices of the tokens, one after the other, which bounds
        # the size of the permuted / exchanged buffers (paddleformers/transformers/qwen3_moe/modeling.py:447-540)
        sub = int(getattr(self.config, "moe_subbatch_token_num_before_dispatch", 0) or 0)
        if sub > 0 and x2d.shape[0] > sub:
            outs, auxes = [], []
            # the peer-memory exchange keeps ONE exchange per layer alive for the backward pass; several sub-batches per
            # layer therefore go through the all-to-all path
            self._single_exchange_buffers_busy = True
            try:
                for piece in x2d.split(sub, dim=0):
                    outs.append(self._forward_tokens(piece))
                    if self.last_aux_loss is not None:
                        auxes.append(self.last_aux_loss)
            finally:
                self._single_exchange_buffers_busy = False
            self.last_aux_loss = torch.stack(auxes).mean() if auxes else None
            return torch.cat(outs, dim=0)
        return self._forward_tokens(x2d)

    def _forward_tokens(self, x2d: torch.Tensor) -> torch.Tensor:
        T, H = x2d.shape
        idx, w, aux = self.gate(x2d)
        # PFB_FUSED_EP_SINGLE=1 sends a single expert-parallel rank through the peer-memory exchange as well (the kernels then
        # exchange with themselves): the way to exercise the exchange, its buffers and their pipeline slots on few GPUs
        if self.ep > 1 or (x2d.is_cuda and os.environ.get("PFB_FUSED_EP_SINGLE", "0") == "1"
                           and getattr(self.config, "moe_token_dispatcher_type", "fused") == "fused"):
            from ..parallel.expert_parallel import ep_moe_forward

            assert not getattr(self.config, "moe_scale_expert_input", False), \
                "routing weights on the expert input are implemented for expert-parallel degree 1"
            y = ep_moe_forward(self, x2d, idx, w)
        elif getattr(self.config, "moe_scale_expert_input", False):
            # the routing weight multiplies what the expert READS (Llama 4): every (token, slot) pair becomes its own scaled
            # row, and the outputs are summed with weight one
            dest, block_expert, rows, counts = build_dispatch_plan(idx, self.experts.num_local, 0)
            pairs = (x2d[:, None, :] * w[:, :, None].to(x2d.dtype)).reshape(T * idx.shape[1], H)
            xr = _PermuteFn.apply(pairs, dest, 1, rows)
            yr = self.experts(xr, block_expert, counts)
            y = unpermute_combine(yr, dest, torch.ones_like(w), T)
        else:
            dest, block_expert, rows, counts = build_dispatch_plan(idx, self.experts.num_local, 0)
            xr = _PermuteFn.apply(x2d, dest, idx.shape[1], rows)
            yr = self.experts(xr, block_expert, counts)
            y = unpermute_combine(yr, dest, w, T)
        if self.shared_experts is not None:
            shared = self.shared_experts(x2d)
            if self.shared_expert_gate is not None:
                shared = shared * torch.sigmoid(TF.linear(x2d, self.shared_expert_gate.weight)).to(shared.dtype)
            y = y + shared
        if aux is not None and self._token_slices > 1:
            # under sequence parallelism every tensor-parallel rank adds the balance term of ITS token slice and the router
            # gradients of the ranks are summed: each term counts 1 / tp, so that together they weigh as much as the one
            # term of the unsplit batch
            aux = aux / self._token_slices
        self.last_aux_loss = aux.detach() if aux is not None else None
        if aux is not None:
            y = AddAuxiliaryLoss.apply(y, aux)
        return y


class ModalityMoELayer(nn.Module):
    """Two isolated expert groups, one serving text tokens and one serving image / video tokens, each with its own router
    and expert width, plus shared experts that see every token (ERNIE-4.5-VL;
    paddleformers/transformers/ernie4_5_moe_vl/model/modeling_moe_vl.py). ``vision_rows`` (bool [tokens], set by the model
    before the layers run; None = text only) says which rows go to the vision group."""

    def __init__(self, config, dtype=None, device=None):
        super().__init__()
        import copy

        text_cfg, vis_cfg = copy.copy(config), copy.copy(config)
        text_cfg.n_shared_experts = vis_cfg.n_shared_experts = 0
        vis_cfg.moe_intermediate_size = int(config.moe_vision_intermediate_size)
        self.text_moe = MoELayer(text_cfg, dtype=dtype, device=device)
        self.vision_moe = MoELayer(vis_cfg, dtype=dtype, device=device)
        self.shared_experts = None
        if config.n_shared_experts:
            self.shared_experts = DenseMLP(config.hidden_size, config.moe_intermediate_size * config.n_shared_experts, config,
                                           tp=False, dtype=dtype, device=device)
        self.ep = get_parallel_state().degrees.ep
        self.vision_rows: Optional[torch.Tensor] = None
        self.last_aux_loss = None

    def forward(self, x2d: torch.Tensor) -> torch.Tensor:
        vis = self.vision_rows
        if vis is None and self.ep == 1:
            y = self.text_moe(x2d)
        else:
            if vis is None:
                vis = torch.zeros(x2d.shape[0], dtype=torch.bool, device=x2d.device)
            assert vis.numel() == x2d.shape[0], "one modality flag per token row"
            y = torch.zeros_like(x2d)
            for rows, moe in ((torch.nonzero(~vis)[:, 0], self.text_moe), (torch.nonzero(vis)[:, 0], self.vision_moe)):
                # under expert parallelism both groups run on every rank (their exchanges are collective), also on no rows
                if rows.numel() or self.ep > 1:
                    y = y.index_add(0, rows, moe(x2d.index_select(0, rows)))
        aux = [m.last_aux_loss for m in (self.text_moe, self.vision_moe) if m.last_aux_loss is not None]
        self.last_aux_loss = torch.stack(aux).sum() if aux else None
        if self.shared_experts is not None:
            y = y + self.shared_experts(x2d)
        return y
