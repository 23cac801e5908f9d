"""Expert-parallel token dispatch / combine.

Two implementations of the same exchange:

* ``alltoall`` — the NCCL baseline: counts are exchanged first, the split sizes are read on the host, tokens travel
  with ``all_to_all_single`` (the reference's naive path, paddleformers/nn/moe_deepep/moe_communication.py:138-200,
  which also synchronises with the host for the split sizes).
* ``fused`` — the peer-memory path of ``parallel.fused_collectives``: every rank writes its routed rows straight into
  the destination rank's expert-sorted receive buffer over NVLink from inside one kernel, with device-side slot
  counters and no host synchronisation (the role DeepEP plays for the reference,
  paddleformers/transformers/fused_a2a.py:81-178). Selected when a symmetric workspace is available.

Both return rows grouped by local expert and padded to 128-row segments, ready for the grouped GEMM.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..nn import moe as moe_mod
from .topology import get_parallel_state


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits: List[int], in_splits: List[int], group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits,
                               group=ctx.group)
        return out, None, None, None


def all_to_all(x, out_splits, in_splits, group):
    return _AllToAll.apply(x, out_splits, in_splits, group)


def ep_moe_forward(layer, x2d: torch.Tensor, idx: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Routed-expert part of an MoE layer under expert parallelism. x2d: [T, H]; idx, w: [T, k]."""
    ps = get_parallel_state()
    dispatcher = getattr(layer.config, "moe_token_dispatcher_type", "fused")
    # the fused path keeps the receive and output buffers of a layer per micro-batch slot; the pipeline engine assigns the
    # slots (parallel.fused_ep.SlotAllocator), without pipeline parallelism there is one
    if dispatcher == "fused" and not getattr(layer, "_single_exchange_buffers_busy", False):
        from . import fused_collectives as fc

        ws = fc.get_ep_workspace(ps, x2d, layer)
        if ws is not None:
            return fc.fused_ep_moe_forward(ws, layer, x2d, idx, w)
    return _alltoall_moe_forward(layer, x2d, idx, w, ps)


def _alltoall_moe_forward(layer, x2d, idx, w, ps):
    group = ps.group("ep")
    ep = ps.degrees.ep
    E_local = layer.experts.num_local
    T, H = x2d.shape
    k = idx.shape[1]
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)                  # pairs sorted by global expert id (= by rank)
    send_counts = torch.bincount(flat_e, minlength=ep * E_local).view(ep, E_local)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    # the NCCL path needs the split sizes on the host (one synchronisation per layer)
    sizes = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()
    send_splits, recv_splits = sizes[0].tolist(), sizes[1].tolist()
    src_tok = order // k
    x_send = x2d[src_tok]
    x_recv = all_to_all(x_send, recv_splits, send_splits, group)
    # received rows are ordered (source rank, local expert): regroup by expert into 128-row padded segments
    rc = recv_counts.reshape(-1)
    recv_expert = torch.repeat_interleave(torch.arange(E_local, device=x2d.device).repeat(ep), rc,
                                          output_size=int(sum(recv_splits)))
    if recv_expert.numel() == 0:
        y_recv = x_recv
    else:
        dest, block_expert, rows, counts = moe_mod.build_dispatch_plan(recv_expert[:, None], E_local, 0)
        xr = moe_mod._PermuteFn.apply(x_recv, dest, 1, rows)
        yr = layer.experts(xr, block_expert, counts)
        y_recv = yr[dest]
    y_back = all_to_all(y_recv, send_splits, recv_splits, group)
    weights = w.reshape(-1)[order].to(y_back.dtype)
    out = torch.zeros((T, H), dtype=torch.float32, device=x2d.device)
    out = out.index_add(0, src_tok, (y_back * weights[:, None]).float())
    return out.to(x2d.dtype)
