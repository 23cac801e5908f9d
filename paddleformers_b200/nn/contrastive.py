"""Contrastive objectives for embedding models (retrieval / sentence embeddings).

* ``SimpleContrastiveLoss`` - InfoNCE over in-batch negatives: query i is matched with passage ``i * group`` among all
  passages (``group`` = passages per query: the positive followed by its hard negatives), scores divided by a temperature
  (paddleformers/transformers/contrastive_loss.py:21-38).
* ``MatryoshkaContrastiveLoss`` - the same loss summed over prefixes of the embedding, each prefix re-normalised, so that
  truncated embeddings stay useful (:41-65).
* ``InfClLoss`` / ``MatryoshkaInfClLoss`` - the same objective computed in column tiles with an online log-sum-exp, so that
  the [queries, passages] score matrix is never held; the backward recomputes the tiles. The reference delegates this to an
  external Triton kernel (:68-152); here it is a chunked autograd function, exact up to fp32 rounding.
* ``gather_with_gradient`` - all-gather of representations over the data-parallel ranks that keeps the local slice
  differentiable, so that every rank contrasts against the whole global batch
  (paddleformers/transformers/embedding_utils.py:19-51).
* ``pool_embeddings`` - last-token or mean pooling of decoder hidden states followed by L2 normalisation.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as TF


def _targets(q: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
    group = p.shape[0] // q.shape[0]
    return torch.arange(q.shape[0], device=q.device, dtype=torch.long) * group


class SimpleContrastiveLoss(nn.Module):
    def __init__(self, embedding_temperature: float = 0.02):
        super().__init__()
        self.temperature = float(embedding_temperature)

    def forward(self, q_reps: torch.Tensor, p_reps: torch.Tensor) -> torch.Tensor:
        scores = (q_reps.float() @ p_reps.float().t()) / self.temperature
        return TF.cross_entropy(scores, _targets(q_reps, p_reps))


class _ChunkedInfoNCE(torch.autograd.Function):
    """mean_i [ logsumexp_j(q_i . p_j / t) - q_i . p_target(i) / t ] with the passages visited ``chunk`` columns at a time."""

    @staticmethod
    def forward(ctx, q, p, target, inv_t: float, chunk: int):
        qf, pf = q.float(), p.float()
        n = qf.shape[0]
        m = torch.full((n,), float("-inf"), device=q.device)
        s = torch.zeros(n, device=q.device)
        for lo in range(0, pf.shape[0], chunk):
            sc = (qf @ pf[lo:lo + chunk].t()) * inv_t
            m_new = torch.maximum(m, sc.max(dim=1).values)
            s = s * torch.exp(m - m_new) + torch.exp(sc - m_new[:, None]).sum(dim=1)
            m = m_new
        lse = m + torch.log(s)
        pos = (qf * pf[target]).sum(-1) * inv_t
        ctx.save_for_backward(q, p, target, lse)
        ctx.inv_t, ctx.chunk = inv_t, chunk
        return (lse - pos).mean()

    @staticmethod
    def backward(ctx, g):
        q, p, target, lse = ctx.saved_tensors
        qf, pf = q.float(), p.float()
        n = qf.shape[0]
        coef = g.float() * ctx.inv_t / n
        dq = torch.zeros_like(qf)
        dp = torch.zeros_like(pf)
        for lo in range(0, pf.shape[0], ctx.chunk):
            blk = pf[lo:lo + ctx.chunk]
            prob = torch.exp((qf @ blk.t()) * ctx.inv_t - lse[:, None])        # softmax columns of this tile
            dq += prob @ blk
            dp[lo:lo + ctx.chunk] += prob.t() @ qf
        dq -= pf[target]
        dp.index_add_(0, target, -qf)
        return (dq * coef).to(q.dtype), (dp * coef).to(p.dtype), None, None, None


class InfClLoss(nn.Module):
    def __init__(self, embedding_temperature: float = 0.02, chunk: int = 4096):
        super().__init__()
        self.temperature, self.chunk = float(embedding_temperature), int(chunk)

    def forward(self, q_reps, p_reps):
        return _ChunkedInfoNCE.apply(q_reps, p_reps, _targets(q_reps, p_reps), 1.0 / self.temperature, self.chunk)


class _Matryoshka(nn.Module):
    def __init__(self, base: nn.Module, dims: Optional[List[int]]):
        super().__init__()
        self.base, self.dims = base, list(dims or [])

    def forward(self, q_reps, p_reps):
        if not self.dims:
            return self.base(q_reps, p_reps)
        loss = 0.0
        for d in self.dims:
            loss = loss + self.base(TF.normalize(q_reps[:, :d].float(), dim=-1), TF.normalize(p_reps[:, :d].float(), dim=-1))
        return loss


class MatryoshkaContrastiveLoss(_Matryoshka):
    def __init__(self, embedding_temperature: float = 0.02, embedding_matryoshka_dims: Optional[List[int]] = None):
        super().__init__(SimpleContrastiveLoss(embedding_temperature), embedding_matryoshka_dims)


class MatryoshkaInfClLoss(_Matryoshka):
    def __init__(self, embedding_temperature: float = 0.02, embedding_matryoshka_dims: Optional[List[int]] = None, chunk: int = 4096):
        super().__init__(InfClLoss(embedding_temperature, chunk), embedding_matryoshka_dims)


class _GatherKeepLocal(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x.contiguous(), group=group)
        ctx.rank, ctx.rows = dist.get_rank(group), x.shape[0]
        return torch.cat(parts, dim=0)

    @staticmethod
    def backward(ctx, g):
        # every rank computes the loss of ITS queries against all passages: the gradient w.r.t. a passage is the sum of
        # what all ranks' losses contribute to it
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g[ctx.rank * ctx.rows:(ctx.rank + 1) * ctx.rows], None


def gather_with_gradient(x: Optional[torch.Tensor], group=None) -> Optional[torch.Tensor]:
    """Concatenate ``x`` over the ranks of ``group`` (default: all ranks) in rank order. The result is differentiable: a
    rank's slice receives the sum of the gradients that all ranks computed for it. Equal row counts on all ranks."""
    if x is None or not dist.is_initialized() or dist.get_world_size(group) <= 1:
        return x
    return _GatherKeepLocal.apply(x, group)


def pool_embeddings(hidden: torch.Tensor, attention_mask: Optional[torch.Tensor] = None, pooling: str = "last",
                    normalize: bool = True) -> torch.Tensor:
    """hidden [B, S, H] -> [B, H]: the hidden state of the last real token (``pooling="last"``; right- or left-padded
    rows both work), or the mean over real tokens (``"mean"``)."""
    B, S, _ = hidden.shape
    mask = torch.ones(B, S, dtype=torch.bool, device=hidden.device) if attention_mask is None else attention_mask.bool()
    if pooling == "last":
        idx = (mask.long() * torch.arange(S, device=hidden.device)[None]).argmax(dim=1)
        out = hidden[torch.arange(B, device=hidden.device), idx]
    elif pooling == "mean":
        out = (hidden * mask[..., None].to(hidden.dtype)).sum(1) / mask.sum(1, keepdim=True).clamp(min=1).to(hidden.dtype)
    else:
        raise ValueError(f"unknown pooling {pooling!r} (last, mean)")
    return TF.normalize(out.float(), dim=-1) if normalize else out
