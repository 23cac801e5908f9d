"""Expert-parallel MoE exchange over NVLink peer memory: dispatch and combine without NCCL and without host reads.

The NCCL path (``parallel.expert_parallel._alltoall_moe_forward``) reads the split sizes back to the host once per
layer, which serialises the step and cannot be captured in a CUDA graph. Here the receive buffer has a static capacity
and the whole exchange is stream-ordered device work (the role DeepEP's ``Buffer.dispatch`` / ``combine`` play for the
reference, paddleformers/transformers/fused_a2a.py:81-178 and paddleformers/nn/moe_deepep/moe_communication.py:31-137):

1. ``ep_exchange``   counts -> every destination; receive-side layout (expert segments padded to 128 rows, block ->
                     expert table, per-expert row table) and per-source slot offsets -> every source.
2. ``ep_push_rows``  each routed pair's row goes straight into its slot of the destination's receive buffer.
3. grouped expert GEMMs on the receive buffer, output written into a peer-visible buffer.
4. ``ep_pull_rows``  each source reads its k rows back and forms the weighted sum.

The backward pass mirrors it: the combine's backward pushes ``w * dout`` rows; the routing-weight gradient is formed on
the expert's side (a dot product of each received gradient row with the expert output beside it, 4 bytes per pair
fetched back; ``PFB_EP_LOCAL_DOTS=0`` re-reads the expert outputs remotely instead); the dispatch's backward pulls the
expert input gradients.

Buffers. Per MoE layer and micro-batch in flight: the receive buffer (it is the saved activation of the expert GEMMs) and
the expert output buffer (read again in the backward pass). Without pipeline parallelism one micro-batch is in flight;
a pipeline schedule keeps several between their forward and backward passes, so the engine gives every micro-batch a
slot (``set_micro_batch_slot``, ``SlotAllocator``) and a layer keeps one buffer pair per slot. Per workspace: one gradient receive buffer and one input-gradient buffer;
they can be shared by all layers because a rank cannot start the next layer's exchange before every peer has finished
reading this layer's buffers (each step of the protocol waits for a flag from every peer). Flags are epoch-valued.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from .fused_collectives import SymmetricArena, _Region

FLAG_COUNTS, FLAG_OFFSETS, FLAG_ROWS, FLAG_Y, FLAG_DY, FLAG_DX, FLAG_RD = 0, 1, 2, 3, 4, 5, 6
_MAX_RANKS = 8
STATS = {"dispatch": 0, "combine": 0}


def capacity_rows(tokens: int, top_k: int, ep: int, num_local: int, factor: float) -> int:
    """Rows of the receive buffer: ``factor`` x the balanced share (every rank sends tokens*top_k pairs, so a balanced
    rank receives tokens*top_k) plus one padding block per local expert."""
    body = int(tokens * top_k * factor)
    return ((body + 127) // 128 + num_local) * 128


class EPWorkspace:
    def __init__(self, ps, T: int, H: int, top_k: int, num_local: int):
        self.ps = ps
        self.group = ps.group("ep")
        self.ep = ps.degrees.ep
        self.rank = ps.rank_in("ep")
        self.EL = num_local
        self.T, self.H, self.k = T, H, top_k
        assert self.ep <= _MAX_RANKS and num_local <= 128
        self.factor = float(os.environ.get("PFB_EP_CAPACITY", "1.5"))
        self.cap = capacity_rows(T, top_k, self.ep, num_local, self.factor)
        self.arena = SymmetricArena(self.group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.table = _Region(self.arena, (2 * self.ep * num_local + 8 * _MAX_RANKS,), torch.int32)
        self.dy = _Region(self.arena, (self.cap, H), torch.bfloat16)
        self.dxr = _Region(self.arena, (self.cap, H), torch.bfloat16)
        self.rowdots = _Region(self.arena, (self.cap,), torch.float32)     # <expert output row, weighted gradient row>
        self.local_dots = os.environ.get("PFB_EP_LOCAL_DOTS", "1") != "0"
        self.fwd_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.bwd_epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.done = torch.zeros(1, dtype=torch.int32, device=dev)
        self.total_rows = torch.zeros(1, dtype=torch.int32, device=dev)

    def layer_buffers(self) -> dict:
        return {"x_recv": _Region(self.arena, (self.cap, self.H), torch.bfloat16),
                "y": _Region(self.arena, (self.cap, self.H), torch.bfloat16)}

    # thin wrappers -------------------------------------------------------------------------------------------
    def wait(self, slot: int, epoch):
        torch.ops.pfb200.ep_wait_flag(self.table.peer_ptrs, self.rank, self.ep, self.EL, slot, epoch)

    def signal(self, slot: int, epoch):
        torch.ops.pfb200.ep_signal_flag(self.table.peer_ptrs, self.rank, self.ep, self.EL, slot, epoch)

    def push(self, x, plan, scale, region: _Region, slot: int, epoch, slots_from_table: bool):
        torch.ops.pfb200.ep_push_rows(x, plan["idx"], plan["rank_in_expert"], scale, self.table.peer_ptrs, plan["pair_slot"],
                                      region.peer_ptrs, self.k, self.EL, self.ep, self.cap, self.rank, slot, epoch, self.done,
                                      slots_from_table)

    def pull(self, out, plan, w, g, dots, region: _Region):
        torch.ops.pfb200.ep_pull_rows(out, plan["idx"], plan["pair_slot"], w, g, dots, region.peer_ptrs, self.table.peer_ptrs,
                                      self.T, self.k, self.H, self.EL, self.ep, self.cap)


_WS: Dict[tuple, EPWorkspace] = {}
_SLOT = 0


def set_micro_batch_slot(slot: int) -> None:
    """Buffer slot of the micro-batch whose forward (or recomputing backward) pass runs next on this rank."""
    global _SLOT
    _SLOT = int(slot)


class SlotAllocator:
    """Hands every micro-batch a buffer slot for the time between its first forward and its last backward chunk on this
    stage; freed slots are reused, so the number of slots equals the schedule's maximum of micro-batches in flight."""

    def __init__(self, chunks_per_micro_batch: int = 1):
        self.chunks = chunks_per_micro_batch
        self.free: list = []
        self.slot_of: Dict[int, int] = {}
        self.left: Dict[int, int] = {}
        self.high_water = 0

    def acquire(self, mb: int) -> int:
        if mb not in self.slot_of:
            self.slot_of[mb] = self.free.pop() if self.free else self.high_water
            if self.slot_of[mb] == self.high_water:
                self.high_water += 1
            self.left[mb] = self.chunks
        return self.slot_of[mb]

    def backward_done(self, mb: int) -> None:
        self.left[mb] -= 1
        if self.left[mb] == 0:
            self.free.append(self.slot_of.pop(mb))
            del self.left[mb]


def dropped_pairs(reset: bool = True) -> int:
    """Routed (token, expert) pairs dropped on this rank since the last reset because a destination's receive buffer
    (``PFB_EP_CAPACITY`` x the balanced share, default 1.5) was full. Synchronises the current stream. With
    ``PFB_EP_OVERFLOW=error`` a non-zero count raises instead: use it when dropping must not pass silently."""
    if not torch.cuda.is_available() or not hasattr(torch.ops.pfb200, "read_drop_count"):
        return 0
    n = int(torch.ops.pfb200.read_drop_count(reset))
    if n and os.environ.get("PFB_EP_OVERFLOW", "drop") == "error":
        raise RuntimeError(f"expert-parallel dispatch dropped {n} routed pairs: raise PFB_EP_CAPACITY (now "
                           f"{os.environ.get('PFB_EP_CAPACITY', '1.5')}) or balance the router")
    return n


def get_workspace(ps, x2d, layer):
    if x2d.dtype != torch.bfloat16 or x2d.shape[1] % 8 != 0 or ps.degrees.ep > _MAX_RANKS or os.environ.get("PFB_FUSED_EP", "1") == "0":
        return None
    T, H = x2d.shape
    k = layer.gate.top_k
    key = (id(ps), T, H, k, layer.experts.num_local)
    if key not in _WS:
        _WS[key] = EPWorkspace(ps, T, H, k, layer.experts.num_local)
    return _WS[key]


def make_plan(ws: EPWorkspace, idx: torch.Tensor, routed: dict = None) -> dict:
    """Device-side bookkeeping of one exchange: per-expert pair counts and every pair's rank inside its expert (stable
    in pair order), with no host read. ``routed`` is what the routing kernel already produced for these indices
    (``TopkRouter.last_plan``); without it the ranks come from a stable sort."""
    from ..nn.moe import count_ids

    E = ws.ep * ws.EL
    flat = idx.reshape(-1).contiguous()
    dev = flat.device
    if routed is not None and routed.get("idx") is idx and routed["counts"].numel() == E:
        counts, rank_in_expert = routed["counts"], routed["rank_in_expert"]
    else:
        counts = count_ids(flat, E)
        order = torch.argsort(flat, stable=True)
        first = torch.cumsum(counts, 0) - counts
        rank_sorted = torch.arange(flat.numel(), device=flat.device) - first[flat[order]]
        rank_in_expert = torch.empty_like(rank_sorted)
        rank_in_expert[order] = rank_sorted
    return {"idx": flat, "counts": counts.to(torch.int32), "rank_in_expert": rank_in_expert.to(torch.int32),
            "pair_slot": torch.empty(flat.numel(), dtype=torch.int32, device=dev),
            "block_expert": torch.empty(ws.cap // 128, dtype=torch.int32, device=dev),
            "expert_rows": torch.empty((ws.EL, 2), dtype=torch.int32, device=dev),
            "expert_tot": torch.empty(ws.EL, dtype=torch.int32, device=dev)}


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2d, ws, bufs, plan):
        ws.push(x2d.contiguous(), plan, None, bufs["x_recv"], FLAG_ROWS, ws.fwd_epoch, True)
        ws.wait(FLAG_ROWS, ws.fwd_epoch)
        ctx.ws, ctx.plan = ws, plan
        ctx.shape = x2d.shape
        STATS["dispatch"] += 1
        return bufs["x_recv"].tensor.detach()      # a fresh tensor object per call: autograd attaches this call's graph to it

    @staticmethod
    def backward(ctx, g):
        ws, plan = ctx.ws, ctx.plan
        # g: gradient of the receive buffer rows, produced by the expert backward which has consumed ws.dy by now
        if g.data_ptr() != ws.dxr.tensor.data_ptr():     # the expert backward normally writes straight into the buffer
            ws.dxr.tensor.copy_(g)
        ws.signal(FLAG_DX, ws.bwd_epoch)
        ws.wait(FLAG_DX, ws.bwd_epoch)
        dx = torch.empty(ctx.shape, dtype=torch.bfloat16, device=g.device)
        ws.pull(dx, plan, None, None, None, ws.dxr)
        return dx, None, None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_rows, w, ws, bufs, plan):
        # y_rows is bufs["y"].tensor, written by the expert GEMM that precedes this call in stream order
        ws.signal(FLAG_Y, ws.fwd_epoch)
        ws.wait(FLAG_Y, ws.fwd_epoch)
        out = torch.empty((ws.T, ws.H), dtype=torch.bfloat16, device=y_rows.device)
        wf = w.reshape(-1).float().contiguous()
        ws.pull(out, plan, wf, None, None, bufs["y"])
        ctx.ws, ctx.plan, ctx.bufs = ws, plan, bufs
        ctx.save_for_backward(wf)
        ctx.w_shape, ctx.w_dtype = w.shape, w.dtype
        STATS["combine"] += 1
        return out

    @staticmethod
    def backward(ctx, dout):
        ws, plan, bufs = ctx.ws, ctx.plan, ctx.bufs
        (wf,) = ctx.saved_tensors
        dout = dout.contiguous()
        ws.bwd_epoch.add_(1)
        # the gradient buffer is shared by all layers: this layer's padding rows hold older rows and must read as zero in
        # the weight-gradient GEMMs; only they are cleared (peers write the received rows only, so this may overlap their pushes)
        torch.ops.pfb200.ep_zero_padding(ws.dy.tensor, plan["expert_rows"], plan["expert_tot"], ws.EL)
        ws.push(dout, plan, wf, ws.dy, FLAG_DY, ws.bwd_epoch, False)   # reuses the slots recorded in the forward pass
        dots = torch.empty(wf.numel(), dtype=torch.float32, device=dout.device)
        if ws.local_dots:
            # Routing-weight gradient <expert output row, dout> formed where the rows are: once every peer's weighted
            # gradient rows (w * dout) have landed, this rank takes the dot product of each of its rows with the expert
            # output beside it (local memory) and the sources fetch 4 bytes per pair and divide by w, instead of reading
            # the expert outputs (4 KB per pair) across NVLink a second time.
            ws.wait(FLAG_DY, ws.bwd_epoch)
            torch.ops.pfb200.ep_row_dots(bufs["y"].tensor, ws.dy.tensor, ws.rowdots.tensor, plan["expert_rows"], ws.EL)
            ws.signal(FLAG_RD, ws.bwd_epoch)
            ws.wait(FLAG_RD, ws.bwd_epoch)
            torch.ops.pfb200.ep_pull_scalars(dots, plan["idx"], plan["pair_slot"], wf, ws.rowdots.peer_ptrs, ws.EL, ws.ep, ws.cap)
        else:
            ws.pull(None, plan, None, dout, dots, bufs["y"])
            ws.wait(FLAG_DY, ws.bwd_epoch)
        return ws.dy.tensor.detach(), dots.view(ctx.w_shape).to(ctx.w_dtype), None, None, None


def moe_forward(ws: EPWorkspace, layer, x2d, idx, w):
    """Routed-expert output [T, H] of ``layer`` for tokens x2d with routing (idx, w), experts spread over the ep group."""
    by_slot = getattr(layer, "_ep_bufs", None)
    if by_slot is None:
        by_slot = layer._ep_bufs = {}
    bufs = by_slot.get(_SLOT)
    if bufs is None or bufs["x_recv"].tensor.shape != (ws.cap, ws.H):
        bufs = by_slot[_SLOT] = ws.layer_buffers()
    plan = make_plan(ws, idx, getattr(layer.gate, "last_plan", None))
    ws.fwd_epoch.add_(1)
    torch.ops.pfb200.ep_exchange(ws.table.peer_ptrs, plan["counts"], plan["block_expert"], plan["expert_rows"], ws.total_rows,
                                 ws.rank, ws.ep, ws.EL, ws.fwd_epoch, plan["expert_tot"])
    x_recv = _Dispatch.apply(x2d, ws, bufs, plan)
    y_rows = layer.experts(x_recv, plan["block_expert"], None, out=bufs["y"].tensor.detach(), expert_rows=plan["expert_rows"],
                          grad_rows_out=ws.dxr.tensor)
    return _Combine.apply(y_rows, w, ws, bufs, plan)
