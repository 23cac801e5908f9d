"""Head GEMM + cross entropy with the vocabulary split over the tensor-parallel group.

Per chunk of tokens every rank computes its logits shard, the ranks exchange three scalars per row (max, sum of
exponentials, label logit), and each rank turns its shard into gradients in place and contracts it into dh (summed
over ranks at the end) and its own slice of dW. Same algorithm as the reference's TP-aware fused head + loss
(paddleformers/transformers/tensor_parallel_utils.py:248-304).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as TF

from ..ops import functional as F
from .tensor_parallel import parallel_cross_entropy_stats
from .topology import get_parallel_state


class _VocabParallelLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, weight, labels, ignore_index, scale, need_grad, chunk):
        ps = get_parallel_state()
        group = ps.group("mp")
        rank = ps.coord["mp"]
        Vl, H = weight.shape
        T = h.shape[0]
        dev = h.device
        use_kernels = h.is_cuda and h.dtype == torch.bfloat16
        loss_rows = torch.zeros(T, dtype=torch.float32, device=dev)
        dh = torch.zeros_like(h) if need_grad else None
        mg = getattr(weight, "main_grad", None)
        dw = torch.zeros((Vl, H), dtype=torch.float32, device=dev) if (need_grad and mg is None) else None
        wg = mg.view(Vl, H) if mg is not None else dw
        sc = scale.reshape(1).to(torch.float32)
        vstart = rank * Vl
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            hc, lab = h[s:e], labels[s:e]
            n = e - s
            if use_kernels:
                ops = torch.ops.pfb200
                logits = F.gemm(hc, weight)
                smax, ssum, slab = (torch.empty(n, dtype=torch.float32, device=dev) for _ in range(3))
                dummy = torch.empty(1, dtype=torch.float32, device=dev)
                ops.cross_entropy(logits, lab, dummy, smax, ssum, slab, sc, vstart, ignore_index, 1, False)
                gmax, gsum, glab = parallel_cross_entropy_stats(smax, ssum, slab, group)
                valid = lab != ignore_index
                loss_rows[s:e] = torch.where(valid, torch.log(gsum) + gmax - glab, torch.zeros_like(gsum))
                if need_grad:
                    ops.cross_entropy(logits, lab, dummy, gmax, gsum, slab, sc, vstart, ignore_index, 2, True)
                    F.gemm(logits, weight, out=dh[s:e], b_mn=True)
                    F.gemm(logits, hc, out=wg, a_mn=True, b_mn=True, epi=F.EPI_ACCUM_F32)
            else:
                logits = TF.linear(hc, weight).float()
                smax = logits.max(-1)[0]
                ssum = torch.exp(logits - smax[:, None]).sum(-1)
                local = lab - vstart
                inside = (local >= 0) & (local < Vl) & (lab != ignore_index)
                slab = torch.where(inside, logits.gather(1, local.clamp(0, Vl - 1)[:, None])[:, 0], torch.zeros_like(smax))
                gmax, gsum, glab = parallel_cross_entropy_stats(smax, ssum, slab, group)
                valid = lab != ignore_index
                loss_rows[s:e] = torch.where(valid, torch.log(gsum) + gmax - glab, torch.zeros_like(gsum))
                if need_grad:
                    p = torch.exp(logits - gmax[:, None]) / gsum[:, None]
                    onehot = torch.zeros_like(p)
                    onehot[inside, local[inside]] = 1.0
                    g = ((p - onehot) * valid[:, None] * sc).to(h.dtype)
                    dh[s:e] = g @ weight
                    wg += (g.t() @ hc).float()
        if need_grad:
            dist.all_reduce(dh, group=group)
        ctx.save_for_backward(dh if need_grad else torch.empty(0), dw if dw is not None else torch.empty(0))
        ctx.has_dw = dw is not None
        ctx.wdtype = weight.dtype
        count = (labels != ignore_index).sum()
        ctx.mark_non_differentiable(count)
        return loss_rows.sum() * sc[0], count

    @staticmethod
    def backward(ctx, dloss, _):
        dh, dw = ctx.saved_tensors
        return dh * dloss.to(dh.dtype), (dw * dloss).to(ctx.wdtype) if ctx.has_dw else None, None, None, None, None, None


def vocab_parallel_linear_cross_entropy(h, weight, labels, ignore_index=-100, scale=None, chunk: int = 2048):
    """h: [T, H] (complete tokens, replicated over the tp group); weight: [V/tp, H] local shard."""
    if scale is None:
        scale = torch.ones((), dtype=torch.float32, device=h.device)
    need_grad = torch.is_grad_enabled() and (h.requires_grad or weight.requires_grad)
    return _VocabParallelLinearCE.apply(h.contiguous(), weight, labels.contiguous(), ignore_index, scale, need_grad, chunk)
