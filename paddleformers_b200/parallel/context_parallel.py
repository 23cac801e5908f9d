"""Long-sequence parallelism: context parallel batch slicing, all-gather-KV and ring attention, Ulysses resharding.

* ``get_batch_on_this_cp_rank`` — slices every [B, S, ...] input over the cp group, either contiguously or in the
  zig-zag "dual chunk" layout where rank r holds chunks r and 2*cp-1-r of 2*cp equal chunks so that causal attention
  work is balanced (paddleformers/trainer/trainer.py:2296-2306, ``cp_balance_mode``).
* ``cp_attention`` — attention for a cp-sharded sequence: keys / values are all-gathered over the cp group (the
  default of the reference's provider track) and each rank attends with its own query positions.
* ``ring_attention`` — double-buffered K/V ring with log-sum-exp merging
  (paddleformers/transformers/ring_flash_attention.py:23-170), without the per-step device synchronisation of the
  reference: the next block's exchange is posted before the current block's attention is launched.
* ``ReshardLayer`` / ``split_inputs_sequence_dim`` — Ulysses (segment parallel) all-to-all between sequence-sharded
  and head-sharded layouts (paddleformers/transformers/segment_parallel_utils.py:35-137).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import functional as F
from .topology import ParallelState, get_parallel_state

_SEQ_KEYS = ("input_ids", "labels", "position_ids", "attn_mask_startend_row_indices", "loss_mask")


def _zigzag_index(S: int, cp: int, rank: int, device) -> torch.Tensor:
    c = S // (2 * cp)
    a = torch.arange(rank * c, (rank + 1) * c, device=device)
    b = torch.arange((2 * cp - 1 - rank) * c, (2 * cp - rank) * c, device=device)
    return torch.cat([a, b])


def cp_positions(S: int, cp: int, rank: int, mode: str, device) -> torch.Tensor:
    """Global positions of the tokens held by ``rank``."""
    if mode == "contiguous_allgather":
        per = S // cp
        return torch.arange(rank * per, (rank + 1) * per, device=device)
    return _zigzag_index(S, cp, rank, device)


def _keep_unsliced_for_mtp(batch, out, idx) -> None:
    """Multi-token-prediction heads look k tokens ahead, across slice boundaries: the whole token and label rows (small
    integer tensors) travel with the slice, together with the global position of every local token."""
    if "labels" in batch:
        out["full_input_ids"], out["full_labels"], out["mtp_global_positions"] = batch["input_ids"], batch["labels"], idx


def get_batch_on_this_cp_rank(batch: Dict[str, torch.Tensor], ps: Optional[ParallelState] = None,
                              mode: str = "dualchunk_allgather") -> Dict[str, torch.Tensor]:
    ps = ps or get_parallel_state()
    cp, rank = ps.degrees.cp, ps.coord["cp"]
    if cp == 1:
        return batch
    out = dict(batch)
    S = batch["input_ids"].shape[1]
    assert S % (2 * cp) == 0, f"sequence length {S} must be a multiple of 2*cp = {2 * cp}"
    idx = cp_positions(S, cp, rank, mode, batch["input_ids"].device)
    if batch.get("attn_mask_startend_row_indices") is not None:     # every rank needs the bounds of ALL key columns
        out["full_attn_mask_startend_row_indices"] = batch["attn_mask_startend_row_indices"]
    for k in _SEQ_KEYS:
        if k in batch and isinstance(batch[k], torch.Tensor) and batch[k].dim() >= 2 and batch[k].shape[1] == S:
            out[k] = batch[k].index_select(1, idx)
    if "position_ids" not in batch:
        out["position_ids"] = idx[None].expand(batch["input_ids"].shape[0], -1).contiguous()
    out["cp_global_positions"] = idx
    out["cp_full_seq_len"] = S
    _keep_unsliced_for_mtp(batch, out, idx)
    return out


def split_inputs_sequence_dim(batch: Dict[str, torch.Tensor], ps: Optional[ParallelState] = None) -> Dict[str, torch.Tensor]:
    """Ulysses: every rank of the sep group keeps a contiguous slice of the tokens."""
    ps = ps or get_parallel_state()
    n, r = ps.degrees.sep, ps.coord["sep"]
    if n == 1:
        return batch
    out = dict(batch)
    S = batch["input_ids"].shape[1]
    assert S % n == 0
    per = S // n
    if batch.get("attn_mask_startend_row_indices") is not None:
        out["full_attn_mask_startend_row_indices"] = batch["attn_mask_startend_row_indices"]
    out["cp_full_seq_len"] = S
    _keep_unsliced_for_mtp(batch, out, torch.arange(r * per, (r + 1) * per, device=batch["input_ids"].device))
    for k in _SEQ_KEYS:
        if k in batch and isinstance(batch[k], torch.Tensor) and batch[k].dim() >= 2 and batch[k].shape[1] == S:
            out[k] = batch[k][:, r * per:(r + 1) * per].contiguous()
    if "position_ids" not in batch:
        out["position_ids"] = torch.arange(r * per, (r + 1) * per, device=batch["input_ids"].device)[None].expand(
            batch["input_ids"].shape[0], -1).contiguous()
    return out


class _AllGatherSeq(torch.autograd.Function):
    """All-gather along dim 1 (sequence) forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = group.size()
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=1)

    @staticmethod
    def backward(ctx, g):
        n = ctx.group.size()
        r = dist.get_rank(ctx.group)
        chunks = [c.contiguous() for c in g.chunk(n, dim=1)]
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter(out, chunks, group=ctx.group)
        return out, None


def cp_attention(q, k, v, q_positions: torch.Tensor, S_full: int, mode: str, group, scale=None, kend_full=None,
                 block: int = 4096):
    """q, k, v: [B, S_local, H, D] of this cp rank; ``q_positions``: global positions of the local tokens.
    Keys / values of all ranks are gathered and re-ordered to global order; the local queries attend causally by
    global position (and inside ``kend_full[b, j]`` document bounds when given). The keys are visited in blocks with
    log-sum-exp merging, so the score matrix never exceeds [S_local, block] per head, and blocks that lie entirely in
    the future of every local query are skipped."""
    cp = group.size()
    kg = _AllGatherSeq.apply(k, group)
    vg = _AllGatherSeq.apply(v, group)
    dev = q.device
    # position of every gathered key, then the permutation that sorts keys by global position
    pos_all = torch.cat([cp_positions(S_full, cp, r, mode, dev) for r in range(cp)])
    order = torch.argsort(pos_all)
    kg, vg = kg.index_select(1, order), vg.index_select(1, order)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    out = torch.zeros(q.shape[:3] + (v.shape[-1],), dtype=torch.float32, device=dev)
    lse = torch.full(q.shape[:3], -1e30, dtype=torch.float32, device=dev)
    # the local positions are known on the host from (S_full, cp, rank, mode): no device read is needed for the skip
    q_max = int(max(_host_positions(S_full, cp, dist.get_rank(group), mode)))
    for j0 in range(0, S_full, block):
        if j0 > q_max:
            break
        j1 = min(j0 + block, S_full)
        k_pos = torch.arange(j0, j1, device=dev)
        kend_blk = kend_full[:, j0:j1] if kend_full is not None else None
        blk_out, blk_lse = _block_attention(q, kg[:, j0:j1], vg[:, j0:j1], q_positions, k_pos, scale, kend_blk)
        out, lse = _merge(out, lse, blk_out, blk_lse)
    return out.to(q.dtype)


def _host_positions(S: int, cp: int, rank: int, mode: str):
    if mode == "contiguous_allgather":
        per = S // cp
        return range(rank * per, (rank + 1) * per)
    c = S // (2 * cp)
    return list(range(rank * c, (rank + 1) * c)) + list(range((2 * cp - 1 - rank) * c, (2 * cp - rank) * c))


def _merge(out, lse, blk_out, blk_lse):
    """Numerically stable merge of two partial attention results via their log-sum-exps."""
    new_lse = torch.logaddexp(lse, blk_lse)
    w_old = torch.exp(lse - new_lse).unsqueeze(-1)
    w_new = torch.exp(blk_lse - new_lse).unsqueeze(-1)
    return out * w_old + blk_out * w_new, new_lse


def _block_attention(q, k, v, q_pos, k_pos, scale, kend=None):
    """Returns (out [B,Sq,H,D] fp32, lse [B,Sq,H]) of q against one K/V block with causal masking by position
    (``kend``: [B, Sk] document bounds of the block's keys: key j is visible to query positions < kend[b, j])."""
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    qf = q.permute(0, 2, 1, 3).float()
    kf = k.permute(0, 2, 1, 3).float().repeat_interleave(Hq // Hkv, dim=1)
    vf = v.permute(0, 2, 1, 3).float().repeat_interleave(Hq // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    vis = k_pos[None, :] <= q_pos[:, None]
    if kend is not None:
        vis = vis[None] & (q_pos[None, :, None] < kend[:, None, :])
        s = s.masked_fill(~vis[:, None], float("-inf"))
    else:
        s = s.masked_fill(~vis[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1)).nan_to_num(0.0)
    lse = torch.where(torch.isinf(lse), torch.full_like(lse, -1e30), lse)
    return torch.matmul(p, vf).permute(0, 2, 1, 3), lse.permute(0, 2, 1)


def ring_attention(q, k, v, group, S_full: int, mode: str = "dualchunk_allgather", scale=None):
    """Ring attention over the cp group (forward; differentiable through autograd since every step is built from
    differentiable ops and the exchanged blocks are detached copies re-attached by ``_RingExchange``)."""
    cp = group.size()
    rank = dist.get_rank(group)
    dev = q.device
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    q_pos = cp_positions(S_full, cp, rank, mode, dev)
    out = torch.zeros(q.shape, dtype=torch.float32, device=dev)
    lse = torch.full(q.shape[:3], -1e30, dtype=torch.float32, device=dev)
    kv = torch.stack([k, v])
    for step in range(cp):
        src = (rank - step) % cp
        nxt = _RingExchange.apply(kv, group) if step < cp - 1 else None   # posted before this step's compute
        blk_out, blk_lse = _block_attention(q, kv[0], kv[1], q_pos, cp_positions(S_full, cp, src, mode, dev), scale)
        out, lse = _merge(out, lse, blk_out, blk_lse)
        kv = nxt
    return out.to(q.dtype)


class _RingExchange(torch.autograd.Function):
    """Send to the next rank, receive from the previous one; the backward pass sends gradients the other way."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _ring_shift(x, group, +1)

    @staticmethod
    def backward(ctx, g):
        return _ring_shift(g.contiguous(), ctx.group, -1), None


def _ring_shift(x, group, direction):
    n = group.size()
    r = dist.get_rank(group)
    dst = dist.get_global_rank(group, (r + direction) % n)
    src = dist.get_global_rank(group, (r - direction) % n)
    out = torch.empty_like(x)
    ops = [dist.P2POp(dist.isend, x.contiguous(), dst, group), dist.P2POp(dist.irecv, out, src, group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return out


class ReshardLayer(torch.autograd.Function):
    """Ulysses all-to-all: [B, S/n, H, D] (sequence sharded, all heads) <-> [B, S, H/n, D] (all tokens, head sharded)."""

    @staticmethod
    def forward(ctx, x, group, to_heads: bool):
        ctx.group, ctx.to_heads = group, to_heads
        return _ulysses(x, group, to_heads)

    @staticmethod
    def backward(ctx, g):
        return _ulysses(g.contiguous(), ctx.group, not ctx.to_heads), None, None


def _ulysses(x, group, to_heads):
    n = group.size()
    B, S, H, D = x.shape
    if to_heads:
        inp = x.reshape(B, S, n, H // n, D).permute(2, 0, 1, 3, 4).contiguous()      # [n, B, S/n.., H/n, D]
        out = torch.empty_like(inp)
        dist.all_to_all_single(out, inp, group=group)
        return out.permute(1, 0, 2, 3, 4).reshape(B, n * S, H // n, D)
    inp = x.reshape(B, n, S // n, H, D).permute(1, 0, 2, 3, 4).contiguous()            # [n, B, S/n, H_local, D]
    out = torch.empty_like(inp)
    dist.all_to_all_single(out, inp, group=group)
    return out.permute(1, 2, 0, 3, 4).reshape(B, S // n, n * H, D)
