"""Attention back-ends behind one interface (paddleformers/nn/attention/: ``eager_attention.py:31``,
``sdpa_attention.py:24``, ``flashmask_attention.py:24-76``, ``sink_impl.py:33-220``).

Every back-end takes q [B, S, Hq, D], k / v [B, S, Hkv, D] and optional FlashMask start rows
(``attn_mask_startend_row_indices`` [B, S] or [B, 1, S, 1]: key column j is hidden from query rows >= start[j]) and
returns [B, S, Hq, Dv]:

* ``flashmask`` - the tcgen05 flash kernels on the GPU (causal + document masks with tile skipping);
* ``sdpa``      - ``torch.nn.functional.scaled_dot_product_attention`` with a dense mask rebuilt from the row indices;
* ``eager``     - matmul + softmax in fp32; the only back-end that supports attention sinks (one learned logit per head
  that joins the softmax denominator and absorbs probability mass without contributing a value) and soft-capped scores
  (``softcap * tanh(score / softcap)``).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..ops import functional as F
from .general import GeneralInterface


def _kend(row_indices: Optional[torch.Tensor], B: int, S: int) -> Optional[torch.Tensor]:
    if row_indices is None:
        return None
    return row_indices.reshape(B, -1)[:, :S].to(torch.int32)


def flashmask_attention(q, k, v, attn_mask_startend_row_indices=None, scale=None, causal=True, sinks=None):
    if sinks is not None:
        raise NotImplementedError("attention sinks are only available in the eager back-end")
    B, S = q.shape[:2]
    return F.flash_attention(q, k, v, causal, _kend(attn_mask_startend_row_indices, B, S), scale)


def _dense_mask(kend, B, S, causal, device, kstart=None):
    """bool [B, S(query), S(key)]. ``kstart`` [B, S]: first query row that sees key j; it replaces the causal triangle
    (``kstart[j] = j``) and lets a block of keys be visible to the earlier rows of the same block (prefix-LM and image
    blocks: ``kstart[j]`` = first position of j's block)."""
    i = torch.arange(S, device=device)
    if kstart is not None:
        vis = i[None, :, None] >= kstart[:, None, :].to(i.dtype)
    else:
        vis = (i[None, :] <= i[:, None]) if causal else torch.ones(S, S, dtype=torch.bool, device=device)
        vis = vis[None].expand(B, S, S)
    if kend is not None:
        vis = vis & (i[None, :, None] < kend[:, None, :])
    return vis


def sdpa_attention(q, k, v, attn_mask_startend_row_indices=None, scale=None, causal=True, sinks=None, kstart=None):
    if sinks is not None:
        raise NotImplementedError("attention sinks are only available in the eager back-end")
    B, S, Hq, D = q.shape
    rep = Hq // k.shape[2]
    mask = _dense_mask(_kend(attn_mask_startend_row_indices, B, S), B, S, causal, q.device, kstart)[:, None]
    out = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(rep, 1), v.transpose(1, 2).repeat_interleave(rep, 1),
        attn_mask=mask, scale=scale if scale is not None else 1.0 / math.sqrt(D))
    return out.transpose(1, 2)


def eager_attention(q, k, v, attn_mask_startend_row_indices=None, scale=None, causal=True, sinks=None, softcap=None, kstart=None):
    B, S, Hq, D = q.shape
    rep = Hq // k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    s = torch.einsum("bshd,bthd->bhst", q.float(), k.float().repeat_interleave(rep, 2)) * scale
    if softcap:                                         # Gemma 2: scores squashed into (-cap, cap) before the softmax
        s = torch.tanh(s / softcap) * softcap
    vis = _dense_mask(_kend(attn_mask_startend_row_indices, B, S), B, S, causal, q.device, kstart)[:, None]
    s = s.masked_fill(~vis, float("-inf"))
    if sinks is not None:                               # [Hq] logits: an extra column that takes part in the softmax only
        sink = sinks.float().view(1, Hq, 1, 1).expand(B, Hq, S, 1)
        p = torch.softmax(torch.cat([s, sink], dim=-1), dim=-1)[..., :-1]
    else:
        p = torch.softmax(s, dim=-1)
    out = torch.einsum("bhst,bthd->bshd", p, v.float().repeat_interleave(rep, 2))
    return out.to(q.dtype)


class AttentionInterface(GeneralInterface):
    """``AttentionInterface.get(config._attn_implementation)(q, k, v, ...)``."""


AttentionInterface.register("flashmask", flashmask_attention)
AttentionInterface.register("flash_attention_2", flashmask_attention)
AttentionInterface.register("sdpa", sdpa_attention)
AttentionInterface.register("eager", eager_attention)
