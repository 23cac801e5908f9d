"""Attention backward and the generic (any head-dim) attention path.

``flash_attention_backward`` dispatches to the tcgen05 backward kernel when it is available in the extension
(``torch.ops.pfb200.attn_bwd``) and otherwise to a blocked recomputation written with torch matmuls that uses the
saved log-sum-exp, never materialising more than a [heads, block, S] score slab.

``attention_generic`` serves head dims the tcgen05 kernels do not cover yet (for example MLA's 192/128 split,
paddleformers/transformers/deepseek_v3/modeling.py:542-801): blocked online-softmax attention with the same mask
semantics, differentiable through autograd with per-block recomputation.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

_Q_BLOCK = 1024


def _has_kernel(name: str) -> bool:
    try:
        return hasattr(torch.ops.pfb200, name) and getattr(torch.ops.pfb200, name) is not None
    except Exception:
        return False


def _bwd_options():
    from . import functional as F

    return bool(F._attn_backend.get("deterministic", False)), int(F._attn_backend.get("bwd_heads_per_cta", 0))


def _block_visibility(q0, q1, S_k, causal, kend_b, device):
    """[q1-q0, S_k] boolean visibility for query rows q0..q1 of one batch element."""
    i = torch.arange(q0, q1, device=device)[:, None]
    j = torch.arange(S_k, device=device)[None, :]
    vis = (j <= i) if causal else torch.ones(q1 - q0, S_k, dtype=torch.bool, device=device)
    if kend_b is not None:
        vis = vis & (i < kend_b[None, :S_k])
    return vis


def flash_attention_backward(dout, q, k, v, out, lse, causal, kend, kmin, kmax, scale):
    """dq, dk, dv for out = softmax(mask(q k^T * scale)) v. Shapes: q/dout/out [B,S,Hq,D] (out may be [B*S,Hq,D]),
    k/v [B,S,Hkv,D], lse [B,Hq,S] (natural log)."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    Dv = v.shape[-1]
    dout = dout.reshape(B, S, Hq, Dv)
    out = out.reshape(B, S, Hq, Dv)
    if q.is_cuda and Dv == 128 and (D == 128 or (D == 192 and Hq == Hkv)) and _has_kernel("attn_bwd"):
        dq = torch.empty_like(q)
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        torch.ops.pfb200.attn_bwd(dout.contiguous(), q, k, v, out, lse, dq, dk, dv, B, S, scale, causal, kend, kmin, kmax,
                                  *_bwd_options())
        return dq, dk, dv
    return _blocked_backward(dout, q, k, v, out, lse, causal, kend, scale)


def flash_attention_backward_into(dout, q, k, v, out, lse, causal, kend, kmin, kmax, scale, dq, dk, dv):
    """Same as ``flash_attention_backward`` but writes into caller-provided (possibly strided) dq / dk / dv views."""
    B, S, Hq, D = q.shape
    if q.is_cuda and D == 128 and _has_kernel("attn_bwd"):
        torch.ops.pfb200.attn_bwd(dout.contiguous(), q, k, v, out, lse, dq, dk, dv, B, S, scale, causal, kend, kmin, kmax,
                                  *_bwd_options())
        return
    a, b, c = _blocked_backward(dout, q, k, v, out, lse, causal, kend, scale)
    dq.copy_(a); dk.copy_(b); dv.copy_(c)


def _blocked_backward(dout, q, k, v, out, lse, causal, kend, scale):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    G = Hq // Hkv
    dq = torch.empty_like(q)
    dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
    dv = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
    delta = (dout.float() * out.float()).sum(-1)  # [B,S,Hq]
    for b in range(B):
        kb = k[b].permute(1, 0, 2)  # [Hkv,S,D]
        vb = v[b].permute(1, 0, 2)
        kend_b = kend[b] if kend is not None else None
        for q0 in range(0, S, _Q_BLOCK):
            q1 = min(S, q0 + _Q_BLOCK)
            kv_end = q1 if causal else S
            kv_lo = 0
            if kend_b is not None:
                # keys whose masked-from row is <= q0 are invisible to this block; kend is non-decreasing for
                # document masks, so a prefix can be dropped
                invisible = (kend_b[:kv_end] <= q0)
                kv_lo = int(invisible.to(torch.int32).cumprod(0).sum().item())
            ks, vs = kb[:, kv_lo:kv_end], vb[:, kv_lo:kv_end]
            qb = q[b, q0:q1].permute(1, 0, 2).reshape(Hkv, G, q1 - q0, D)
            dob = dout[b, q0:q1].permute(1, 0, 2).reshape(Hkv, G, q1 - q0, D)
            s = torch.einsum("hgqd,hkd->hgqk", qb, ks).float() * scale
            vis = _block_visibility(q0, q1, kv_end, causal, kend_b, q.device)[:, kv_lo:]
            lse_b = lse[b, :, q0:q1].reshape(Hkv, G, q1 - q0, 1)
            p = torch.exp(s - lse_b).masked_fill(~vis, 0.0)
            pb = p.to(q.dtype)
            dv[b, kv_lo:kv_end] += torch.einsum("hgqk,hgqd->khd", pb, dob).float()
            dp = torch.einsum("hgqd,hkd->hgqk", dob, vs).float()
            dl = delta[b, q0:q1].permute(1, 0).reshape(Hkv, G, q1 - q0, 1)
            ds = (p * (dp - dl) * scale).to(q.dtype)
            dq[b, q0:q1] = torch.einsum("hgqk,hkd->qhgd", ds, ks).reshape(q1 - q0, Hq, D)
            dk[b, kv_lo:kv_end] += torch.einsum("hgqk,hgqd->khd", ds, qb).float()
    return dq, dk.to(k.dtype), dv.to(v.dtype)


class _GenericAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, kend, scale):
        B, S, Hq, Dq = q.shape
        Hkv, Dv = k.shape[2], v.shape[3]
        G = Hq // Hkv
        out = torch.empty((B, S, Hq, Dv), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
        for b in range(B):
            kb = k[b].permute(1, 0, 2)
            vb = v[b].permute(1, 0, 2)
            kend_b = kend[b] if kend is not None else None
            for q0 in range(0, S, _Q_BLOCK):
                q1 = min(S, q0 + _Q_BLOCK)
                kv_end = q1 if causal else S
                qb = q[b, q0:q1].permute(1, 0, 2).reshape(Hkv, G, q1 - q0, Dq)
                s = torch.einsum("hgqd,hkd->hgqk", qb, kb[:, :kv_end]).float() * scale
                vis = _block_visibility(q0, q1, kv_end, causal, kend_b, q.device)
                s = s.masked_fill(~vis, float("-inf"))
                l = torch.logsumexp(s, dim=-1, keepdim=True)
                p = torch.exp(s - l).nan_to_num(0.0).to(q.dtype)
                o = torch.einsum("hgqk,hkd->qhgd", p, vb[:, :kv_end])
                out[b, q0:q1] = o.reshape(q1 - q0, Hq, Dv)
                lse[b, :, q0:q1] = l.reshape(Hq, q1 - q0)
        ctx.save_for_backward(q, k, v, out, lse, kend if kend is not None else torch.empty(0))
        ctx.meta = (causal, scale, kend is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, kend = ctx.saved_tensors
        causal, scale, has_kend = ctx.meta
        B, S, Hq, Dq = q.shape
        Hkv, Dv = k.shape[2], v.shape[3]
        G = Hq // Hkv
        dq = torch.empty_like(q)
        dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
        dv = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
        delta = (dout.float() * out.float()).sum(-1)
        for b in range(B):
            kb = k[b].permute(1, 0, 2)
            vb = v[b].permute(1, 0, 2)
            kend_b = kend[b] if has_kend else None
            for q0 in range(0, S, _Q_BLOCK):
                q1 = min(S, q0 + _Q_BLOCK)
                kv_end = q1 if causal else S
                qb = q[b, q0:q1].permute(1, 0, 2).reshape(Hkv, G, q1 - q0, Dq)
                dob = dout[b, q0:q1].permute(1, 0, 2).reshape(Hkv, G, q1 - q0, Dv)
                s = torch.einsum("hgqd,hkd->hgqk", qb, kb[:, :kv_end]).float() * scale
                vis = _block_visibility(q0, q1, kv_end, causal, kend_b, q.device)
                p = torch.exp(s - lse[b, :, q0:q1].reshape(Hkv, G, q1 - q0, 1)).masked_fill(~vis, 0.0)
                pb = p.to(q.dtype)
                dv[b, :kv_end] += torch.einsum("hgqk,hgqd->khd", pb, dob).float()
                dp = torch.einsum("hgqd,hkd->hgqk", dob, vb[:, :kv_end]).float()
                dl = delta[b, q0:q1].permute(1, 0).reshape(Hkv, G, q1 - q0, 1)
                ds = (p * (dp - dl) * scale).to(q.dtype)
                dq[b, q0:q1] = torch.einsum("hgqk,hkd->qhgd", ds, kb[:, :kv_end]).reshape(q1 - q0, Hq, Dq)
                dk[b, :kv_end] += torch.einsum("hgqk,hgqd->khd", ds, qb).float()
        return dq, dk.to(k.dtype), dv.to(v.dtype), None, None, None


def attention_generic(q, k, v, causal: bool, kend: Optional[torch.Tensor], scale: Optional[float]):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    return _GenericAttnFn.apply(q, k, v, causal, kend, scale)
