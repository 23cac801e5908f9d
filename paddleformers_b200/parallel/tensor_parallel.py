"""Tensor-parallel and sequence-parallel layers.

Column-parallel linears split the output features over the tensor-parallel (mp) group, row-parallel linears split
the input features; with sequence parallel the activations between them are kept sharded over tokens
([T/tp, H]) so the collectives become all-gather (before a column-parallel GEMM) and reduce-scatter (after a
row-parallel GEMM), with the mirrored collective in the backward pass. Same dataflow as the reference's
ColumnSequenceParallelLinear / RowSequenceParallelLinear (paddleformers/transformers/linear_utils.py:27-40) and the
Flux-fused variant of its ERNIE recipe
(paddleformers/cli/train/ernie_pretrain/models/sequence_parallel_utils.py:179-236).

Two execution paths share these modules: the NCCL path below (collective, then GEMM kernel) and the fused
peer-memory kernels of ``parallel.fused_collectives`` when a symmetric-memory workspace is attached.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as F
from .topology import get_parallel_state


def _group_size(group) -> int:
    return group.size() if group is not None else 1


# ---------------------------------------------------------------------------------------------------------------
# collective autograd functions
# ---------------------------------------------------------------------------------------------------------------
def all_gather_tokens(x: torch.Tensor, group) -> torch.Tensor:
    n = _group_size(group)
    if n == 1:
        return x
    out = torch.empty((x.shape[0] * n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def reduce_scatter_tokens(x: torch.Tensor, group) -> torch.Tensor:
    n = _group_size(group)
    if n == 1:
        return x
    out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    return out


class AllGatherOp(torch.autograd.Function):
    """tokens: all-gather forward, reduce-scatter backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_tokens(x, group)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_tokens(g, ctx.group), None


class ReduceScatterOp(torch.autograd.Function):
    """tokens: reduce-scatter forward, all-gather backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return reduce_scatter_tokens(x, group)

    @staticmethod
    def backward(ctx, g):
        return all_gather_tokens(g, ctx.group), None


class ScatterOp(torch.autograd.Function):
    """Keep this rank's token slice (no communication); backward all-gathers."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = _group_size(group)
        if n == 1:
            return x
        r = dist.get_rank(group)
        per = x.shape[0] // n
        return x[r * per:(r + 1) * per].contiguous()

    @staticmethod
    def backward(ctx, g):
        return all_gather_tokens(g, ctx.group), None


class GatherOp(torch.autograd.Function):
    """All-gather tokens forward; backward keeps this rank's slice."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return all_gather_tokens(x, group)

    @staticmethod
    def backward(ctx, g):
        n = _group_size(ctx.group)
        if n == 1:
            return g, None
        r = dist.get_rank(ctx.group)
        per = g.shape[0] // n
        return g[r * per:(r + 1) * per].contiguous(), None


class GatherLastDimOp(torch.autograd.Function):
    """Concatenate the ranks' feature shards (logits of a vocabulary-parallel head) along the last dimension. Every rank then
    computes the same function of the full tensor, so the gradient of the full tensor is the same everywhere and the backward
    pass keeps this rank's shard."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group, ctx.width = group, x.shape[-1]
        n = _group_size(group)
        if n == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        if _group_size(ctx.group) == 1:
            return g, None
        r = dist.get_rank(ctx.group)
        return g[..., r * ctx.width:(r + 1) * ctx.width].contiguous(), None


class AllGatherVarlenOp(torch.autograd.Function):
    """All-gather of token rows when every rank holds a different number of them (the rows that survive a label filter):
    the counts are exchanged first, rows are padded to the largest count for the collective and the padding is dropped.
    Output rows are ordered by rank. Backward keeps this rank's rows, like ``GatherOp``
    (paddleformers/transformers/sequence_parallel_utils.py:68-121)."""

    @staticmethod
    def forward(ctx, x, group):
        n = _group_size(group)
        ctx.group = group
        if n == 1:
            ctx.span = None
            return x
        cnt = torch.tensor([x.shape[0]], dtype=torch.int64, device=x.device)
        cnts = torch.empty(n, dtype=torch.int64, device=x.device)
        dist.all_gather_into_tensor(cnts, cnt, group=group)
        counts = cnts.tolist()
        m = max(max(counts), 1)
        pad = torch.zeros((m,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        pad[:x.shape[0]] = x
        out = torch.empty((n * m,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, pad, group=group)
        r = dist.get_rank(group)
        ctx.span = (sum(counts[:r]), counts[r])
        return torch.cat([out[i * m:i * m + c] for i, c in enumerate(counts)], dim=0)

    @staticmethod
    def backward(ctx, g):
        if ctx.span is None:
            return g, None
        lo, c = ctx.span
        return g[lo:lo + c].contiguous(), None


class CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel linear without SP)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        if _group_size(ctx.group) > 1:
            from . import nvls

            g = nvls.all_reduce_(g.contiguous(), ctx.group)      # NVSwitch multicast kernel for bf16, NCCL otherwise
        return g, None


class ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel linear without SP)."""

    @staticmethod
    def forward(ctx, x, group):
        if _group_size(group) > 1:
            from . import nvls

            x = nvls.all_reduce_(x.contiguous(), group)          # NVSwitch multicast kernel for bf16, NCCL otherwise
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def mark_as_sequence_parallel_parameter(p: torch.nn.Parameter) -> None:
    """Parameters replicated over the tp group but fed token-sharded activations (norm weights, router weights)
    get partial gradients per rank; the trainer all-reduces them over the tp group before the optimizer step
    (paddleformers/trainer/trainer_callback.py:936-963)."""
    p.sequence_parallel = True


# ---------------------------------------------------------------------------------------------------------------
# layers
# ---------------------------------------------------------------------------------------------------------------
class ColumnParallelLinear(nn.Module):
    """y_local = x @ W_local^T; W is [out/tp, in] (with fused ``sections`` every section is split separately).

    ``epilogue="swiglu"`` expects sections == [I, I] and returns silu(gate) * up of the local slice."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, sections: Optional[List[int]] = None,
                 sequence_parallel: bool = False, gather_output: bool = False, epilogue: Optional[str] = None,
                 dtype=None, device=None):
        super().__init__()
        ps = get_parallel_state()
        self.tp = ps.degrees.mp
        self.group = ps.group("mp") if self.tp > 1 else None
        assert out_features % self.tp == 0
        self.in_features, self.out_features = in_features, out_features
        self.sections = sections
        self.sequence_parallel = sequence_parallel and self.tp > 1
        self.gather_output = gather_output
        self.epilogue = epilogue
        self.weight = nn.Parameter(torch.empty(out_features // self.tp, in_features, dtype=dtype, device=device))
        self.weight.shard_spec = ("tp", 0, sections)
        self.bias = nn.Parameter(torch.zeros(out_features // self.tp, dtype=dtype, device=device)) if bias else None
        if self.bias is not None:
            self.bias.shard_spec = ("tp", 0, sections)

    def forward(self, x):
        if self.sequence_parallel and self.bias is None and not self.gather_output:
            from . import fused_collectives as fc

            if x.dim() == 2 and fc.get_tp_workspace() is not None and fc.can_fuse(x, self.weight, self.tp, x.shape[0] * self.tp):
                return fc.fused_column_parallel(x, self.weight, self, swiglu=self.epilogue == "swiglu")
        if self.tp > 1:
            x = AllGatherOp.apply(x, self.group) if self.sequence_parallel else CopyToTP.apply(x, self.group)
        if self.epilogue == "swiglu":
            y = F.linear_swiglu(x, self.weight)
        else:
            y = F.linear(x, self.weight, self.bias)
        if self.gather_output and self.tp > 1:
            parts = [torch.empty_like(y) for _ in range(self.tp)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y


class RowParallelLinear(nn.Module):
    """y = sum_ranks x_local @ W_local^T; W is [out, in/tp]. Output is reduce-scattered over tokens with SP,
    all-reduced otherwise."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, sequence_parallel: bool = False,
                 input_is_parallel: bool = True, dtype=None, device=None):
        super().__init__()
        ps = get_parallel_state()
        self.tp = ps.degrees.mp
        self.group = ps.group("mp") if self.tp > 1 else None
        assert in_features % self.tp == 0
        self.in_features, self.out_features = in_features, out_features
        self.sequence_parallel = sequence_parallel and self.tp > 1
        self.weight = nn.Parameter(torch.empty(out_features, in_features // self.tp, dtype=dtype, device=device))
        self.weight.shard_spec = ("tp", 1, None)
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        if self.bias is not None and self.sequence_parallel:
            mark_as_sequence_parallel_parameter(self.bias)

    def forward(self, x):
        if self.sequence_parallel and x.dim() == 2:
            from . import fused_collectives as fc

            if (fc.get_tp_workspace() is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[0] % (self.tp * 128) == 0
                    and self.out_features % 128 == 0 and x.shape[1] % 8 == 0):
                y = fc.fused_row_parallel(x, self.weight)
                return y + self.bias if self.bias is not None else y
        y = F.linear(x, self.weight)
        if self.tp > 1:
            y = ReduceScatterOp.apply(y, self.group) if self.sequence_parallel else ReduceFromTP.apply(y, self.group)
        if self.bias is not None:
            y = y + self.bias
        return y


class VocabParallelEmbedding(nn.Module):
    """Embedding rows split over the tp group; out-of-shard ids contribute zeros and the partial results are
    summed (all-reduce, or reduce-scatter over tokens when the output feeds a sequence-parallel block)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, sequence_parallel: bool = False, dtype=None, device=None):
        super().__init__()
        ps = get_parallel_state()
        self.tp = ps.degrees.mp
        self.group = ps.group("mp") if self.tp > 1 else None
        self.rank = ps.coord["mp"]
        assert num_embeddings % self.tp == 0, "vocabulary must divide the tensor parallel degree (pad it)"
        self.per = num_embeddings // self.tp
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.sequence_parallel = sequence_parallel and self.tp > 1
        self.weight = nn.Parameter(torch.empty(self.per, embedding_dim, dtype=dtype, device=device))
        self.weight.shard_spec = ("tp", 0, None)

    def forward(self, ids, whole: bool = False):
        """``whole``: all token rows on every rank even under sequence parallelism (for callers that still edit rows by global
        position, e.g. write image features over placeholders, before they cut the token slice)."""
        out = F.embedding(ids, self.weight, vocab_start=self.rank * self.per if self.tp > 1 else 0)
        if self.tp > 1:
            flat = out.reshape(-1, self.embedding_dim)
            if self.sequence_parallel and not whole:
                return ReduceScatterOp.apply(flat, self.group)
            return ReduceFromTP.apply(flat, self.group).view(*ids.shape, self.embedding_dim)
        return out


def parallel_cross_entropy_stats(local_max, local_sum, local_label, group):
    """Combine per-shard (max, sum exp(x - max), label logit) into global softmax statistics
    (paddleformers/transformers/tensor_parallel_utils.py:272-304)."""
    gmax = local_max.clone()
    dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
    gsum = local_sum * torch.exp(local_max - gmax)
    packed = torch.stack([gsum, local_label])
    dist.all_reduce(packed, group=group)
    return gmax, packed[0], packed[1]
