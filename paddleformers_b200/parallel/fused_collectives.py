"""Tensor-parallel linears whose collective runs inside the GEMM kernel over NVLink peer memory.

``fused_column_parallel`` = all-gather(tokens) -> GEMM and ``fused_row_parallel`` = GEMM -> reduce-scatter(tokens), with
the mirrored fused kernel in the backward pass and the gathered activation kept in symmetric memory for the
weight-gradient GEMM (no re-gather, no second copy). They replace the NCCL collective + GEMM pairs of
``parallel.tensor_parallel`` when a ``TPWorkspace`` exists for the tensor-parallel group; the NCCL path stays as the
A/B baseline (``PFB_FUSED_TP=0``).

Buffers (all symmetric, carved from ``SymmetricArena`` chunks so that one handle exchange serves many layers):

* per column-parallel layer: gathered input G [T, K] (doubles as the saved activation), a ready pad [tp], block flags;
* per tensor-parallel group and shape: two reduce-scatter staging buffers [tp, T/tp, N] with their counters, and two
  gathered-gradient buffers for the backward all-gather, used alternately (a rank can never be two fused calls ahead
  of a peer, because finishing a call needs every peer's signal of that call).

The EP dispatch / combine workspace hooks at the bottom are looked up by ``parallel.expert_parallel``.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as F
from .symmetric_memory import SymmetricBuffer
from .topology import get_parallel_state

_ARENA_CHUNK = 1 << 30
STATS = {"ag_gemm": 0, "gemm_rs": 0}


def fused_tp_enabled() -> bool:
    return os.environ.get("PFB_FUSED_TP", "1") != "0"


class SymmetricArena:
    """Bump allocator over symmetric chunks; every rank performs the same allocation sequence, so an (chunk, offset)
    pair names the same region on every rank."""

    def __init__(self, group):
        self.group = group
        self.chunks: List[SymmetricBuffer] = []
        self.used: List[int] = []

    def alloc(self, nbytes: int) -> Tuple[SymmetricBuffer, int]:
        nbytes = (nbytes + 1023) // 1024 * 1024
        for i, ch in enumerate(self.chunks):
            if self.used[i] + nbytes <= ch.nbytes:
                off = self.used[i]
                self.used[i] += nbytes
                return ch, off
        ch = SymmetricBuffer(max(nbytes, _ARENA_CHUNK), self.group)
        self.chunks.append(ch)
        self.used.append(nbytes)
        return ch, 0


CANARY_BYTES = 1024
CANARY_WORD = 0x5AA55AA5
_CANARIES: List[torch.Tensor] = []       # int32 views of the guard words behind every region (PFB_DEBUG_CANARY=1)


def canaries_enabled() -> bool:
    return os.environ.get("PFB_DEBUG_CANARY", "0") == "1"


def check_canaries() -> int:
    """Debug aid for the peer-memory kernels (PFB_DEBUG_CANARY=1): every region of a symmetric arena is followed by 1 KB of
    guard words that no kernel, local or remote, may touch. Returns the number of regions whose guard was overwritten
    (one device synchronisation); 0 when the mode is off."""
    if not _CANARIES:
        return 0
    bad = torch.stack([(c != CANARY_WORD).any() for c in _CANARIES]).sum()
    return int(bad)


class _Region:
    """A tensor inside the arena plus the table of its addresses on every peer."""

    def __init__(self, arena: SymmetricArena, shape, dtype):
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        guard = canaries_enabled()
        payload = (nbytes + 1023) // 1024 * 1024
        buf, off = arena.alloc(payload + CANARY_BYTES if guard else nbytes)
        if guard:
            c = buf.tensor((CANARY_BYTES // 4,), torch.int32, off + payload)
            c.fill_(CANARY_WORD)
            _CANARIES.append(c)
        self.tensor = buf.tensor(shape, dtype, off)
        self.peer_ptrs = torch.tensor([p + off for p in buf.peer_ptrs], dtype=torch.int64)
        self.local_ptr = buf.local_ptr + off


class TPWorkspace:
    def __init__(self, ps=None):
        self.ps = ps or get_parallel_state()
        self.group = self.ps.group("mp")
        self.tp = self.ps.degrees.mp
        self.rank = self.ps.coord["mp"]
        self.arena = SymmetricArena(self.group)
        self._rs: Dict[Tuple[int, int], dict] = {}
        self._bwd_ag: Dict[Tuple[int, int], dict] = {}
        # copy CTAs of the all-gather (each keeps five 32 KB chunks in flight)
        self.n_copy_ctas = int(os.environ.get("PFB_AG_COPY_CTAS", "16" if self.tp >= 8 else "8"))

    def layer_gather_buffers(self, T: int, K: int) -> dict:
        """Persistent buffers of one column-parallel layer."""
        return {"G": _Region(self.arena, (T, K), torch.bfloat16), "ready": _Region(self.arena, (max(self.tp, 8),), torch.int32),
                "blk": torch.zeros(T // 128, dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device())),
                "epoch": torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))}

    def rs_buffers(self, T: int, N: int) -> dict:
        key = (T, N)
        if key not in self._rs:
            self._rs[key] = {"stage": [_Region(self.arena, (T, N), torch.bfloat16) for _ in range(2)],
                             "count": [_Region(self.arena, (max(self.tp, 8),), torch.int32) for _ in range(2)],
                             "epoch": [torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))
                                       for _ in range(2)], "calls": 0}
        return self._rs[key]

    def bwd_gather_buffers(self, T: int, K: int) -> dict:
        key = (T, K)
        if key not in self._bwd_ag:
            self._bwd_ag[key] = {"bufs": [self.layer_gather_buffers(T, K) for _ in range(2)], "calls": 0}
        return self._bwd_ag[key]


_WS: Dict[int, Optional[TPWorkspace]] = {}


def get_tp_workspace() -> Optional[TPWorkspace]:
    ps = get_parallel_state()
    if ps.degrees.mp <= 1 or not fused_tp_enabled() or not torch.cuda.is_available() or not dist.is_initialized():
        return None
    key = id(ps)
    if key not in _WS:
        _WS[key] = TPWorkspace(ps)
    return _WS[key]


def release_workspaces() -> None:
    """Free the symmetric buffers of every tensor-parallel and expert-parallel workspace (collective over their groups:
    every rank must call it at the same point, with no kernel that uses the buffers in flight). Layers keep references
    to their per-layer regions, so drop the model first."""
    from . import fused_ep

    if torch.cuda.is_available():
        torch.cuda.synchronize()
    for ws in list(_WS.values()) + list(fused_ep._WS.values()):
        if ws is None:
            continue
        for ch in ws.arena.chunks:
            ch.close()
        ws.arena.chunks.clear()
        ws.arena.used.clear()
    _WS.clear()
    fused_ep._WS.clear()
    _CANARIES.clear()


# ---------------------------------------------------------------------------------------------------------------
# raw calls
# ---------------------------------------------------------------------------------------------------------------
def _ag_gemm(ws: TPWorkspace, bufs: dict, x_local, weight, b_mn: bool, swiglu: bool):
    G = bufs["G"].tensor
    T, K = G.shape
    R = T // ws.tp
    G[ws.rank * R:(ws.rank + 1) * R].copy_(x_local)
    bufs["epoch"].add_(1)   # device-side counter: a captured graph advances it on every replay
    STATS["ag_gemm"] += 1
    N = weight.shape[1] if b_mn else weight.shape[0]
    out = torch.empty((T, N // 2 if swiglu else N), dtype=torch.bfloat16, device=x_local.device)
    raw = torch.empty((T, N), dtype=torch.bfloat16, device=x_local.device) if swiglu else None
    torch.ops.pfb200.ag_gemm(G, bufs["G"].peer_ptrs, weight, out, raw, F.EPI_SWIGLU_BF16 if swiglu else F.EPI_STORE_BF16, b_mn,
                             bufs["ready"].local_ptr, bufs["ready"].peer_ptrs, bufs["blk"], bufs["epoch"], ws.rank, ws.tp,
                             ws.n_copy_ctas)
    return out, raw, G


def _gemm_rs(ws: TPWorkspace, x, weight, b_mn: bool):
    T = x.shape[0]
    N = weight.shape[1] if b_mn else weight.shape[0]
    st = ws.rs_buffers(T, N)
    par = st["calls"] & 1
    st["calls"] += 1
    st["epoch"][par].add_(1)
    STATS["gemm_rs"] += 1
    out = torch.empty((T // ws.tp, N), dtype=torch.bfloat16, device=x.device)
    torch.ops.pfb200.gemm_rs(x, weight, b_mn, st["stage"][par].peer_ptrs, st["count"][par].peer_ptrs, out, st["epoch"][par],
                             ws.rank, ws.tp)
    return out


def _contig(t):
    return t if (t.stride(-1) == 1 and (t.stride(0) * t.element_size()) % 16 == 0) else t.contiguous()


# ---------------------------------------------------------------------------------------------------------------
# autograd
# ---------------------------------------------------------------------------------------------------------------
class _FusedColumnParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weight, ws, bufs, swiglu):
        out, raw, G = _ag_gemm(ws, bufs, x_local, weight, False, swiglu)
        ctx.ws, ctx.swiglu, ctx.G = ws, swiglu, G
        ctx.save_for_backward(weight, raw if raw is not None else torch.empty(0))
        return out

    @staticmethod
    def backward(ctx, dy):
        weight, raw = ctx.saved_tensors
        ws = ctx.ws
        dy = _contig(dy)
        if ctx.swiglu:
            dy, _ = torch.ops.pfb200.swiglu_bwd(dy.contiguous(), raw, False)
        dw = F._weight_grad(dy, ctx.G, weight)
        dx_local = _gemm_rs(ws, dy, weight, True)
        return dx_local, dw, None, None, None


class _FusedRowParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, ws):
        x2 = _contig(x)
        out = _gemm_rs(ws, x2, weight, False)
        ctx.ws = ws
        ctx.save_for_backward(x2, weight)
        return out

    @staticmethod
    def backward(ctx, dy_local):
        x2, weight = ctx.saved_tensors
        ws = ctx.ws
        T = x2.shape[0]
        H = dy_local.shape[1]
        st = ws.bwd_gather_buffers(T, H)
        bufs = st["bufs"][st["calls"] & 1]
        st["calls"] += 1
        dx, _, Gd = _ag_gemm(ws, bufs, dy_local.contiguous(), weight, True, False)
        dw = F._weight_grad(Gd, x2, weight)
        return dx, dw, None


def fused_column_parallel(x_local, weight, layer, swiglu: bool = False):
    """x_local: [T/tp, K] token shard; weight: [N/tp, K]. Returns [T, N/tp] (or silu(gate)*up of it)."""
    ws = get_tp_workspace()
    T = x_local.shape[0] * ws.tp
    bufs = getattr(layer, "_fused_bufs", None)
    if bufs is None or bufs["G"].tensor.shape != (T, x_local.shape[1]):
        bufs = ws.layer_gather_buffers(T, x_local.shape[1])
        layer._fused_bufs = bufs
    return _FusedColumnParallel.apply(x_local, weight, ws, bufs, swiglu)


def fused_row_parallel(x, weight):
    """x: [T, K/tp]; weight: [N, K/tp]. Returns the token shard [T/tp, N] of the summed product."""
    return _FusedRowParallel.apply(x, weight, get_tp_workspace())


def can_fuse(x, weight, tp: int, tokens_total: int) -> bool:
    return (fused_tp_enabled() and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and tokens_total % (tp * 128) == 0
            and x.shape[1] % 128 == 0 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0 and tp <= 8)


# ---------------------------------------------------------------------------------------------------------------
# expert-parallel workspace hooks
# ---------------------------------------------------------------------------------------------------------------
def get_ep_workspace(ps, x2d, layer):
    """Symmetric workspace of the fused dispatch / combine kernels, or None when they are not available (CPU ranks,
    extension built without them): the caller then uses the NCCL all-to-all path."""
    if not x2d.is_cuda or not hasattr(torch.ops.pfb200, "ep_exchange"):
        return None
    from . import fused_ep

    return fused_ep.get_workspace(ps, x2d, layer)


def fused_ep_moe_forward(ws, layer, x2d, idx, w):
    from . import fused_ep

    return fused_ep.moe_forward(ws, layer, x2d, idx, w)
