"""Context arm of the benchmark: the same Llama-3-8B training step written with stock PyTorch operators only
(``torch.nn.functional.linear`` -> cuBLAS, ``scaled_dot_product_attention``, NCCL all-gather / reduce-scatter for tensor +
sequence parallelism, ``torch.optim.AdamW(fused=True)``). None of this repository's kernels, models or trainer is on this
path. It is NOT the reference implementation (``bench.py --impl reference`` answers for that); it only places the
framework's number next to what the libraries shipped with PyTorch reach on the same box.

What it does and does not do: bf16 parameters and bf16 gradients accumulated by autograd over the micro-batches, AdamW
moments in bf16 (no fp32 master weights and no fp32 gradient accumulation, which the framework's step does carry), no
activation recomputation, global-norm clipping, the same synthetic data, the same timing (barrier + synchronize + CUDA
events, max over ranks).

    python bench.py --impl torch-baseline --gpus 1 --steps 2 --warmup 3
"""
from __future__ import annotations

import json
import math
import os

import torch
import torch.distributed as dist
import torch.nn.functional as TF


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = torch.empty((x.shape[0] * dist.get_world_size(group),) + x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty((g.shape[0] // dist.get_world_size(ctx.group),) + g.shape[1:], dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = torch.empty((x.shape[0] // dist.get_world_size(group),) + x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty((g.shape[0] * dist.get_world_size(ctx.group),) + g.shape[1:], dtype=g.dtype, device=g.device)
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


class Layer(torch.nn.Module):
    def __init__(self, H, I, nq, nkv, D, tp, dev):
        super().__init__()
        self.nq, self.nkv, self.D, self.tp = nq // tp, max(nkv // tp, 1), D, tp
        mk = lambda o, i: torch.nn.Parameter(torch.randn(o, i, device=dev, dtype=torch.bfloat16) * 0.02)
        self.qkv = mk((self.nq + 2 * self.nkv) * D, H)
        self.o = mk(H, self.nq * D)
        self.gu = mk(2 * I // tp, H)
        self.down = mk(H, I // tp)
        self.n1 = torch.nn.Parameter(torch.ones(H, device=dev, dtype=torch.bfloat16))
        self.n2 = torch.nn.Parameter(torch.ones(H, device=dev, dtype=torch.bfloat16))

    def forward(self, x, cos, sin, group, B, S):          # x: [B*S/tp, H] token shard (whole rows when tp == 1)
        h = TF.rms_norm(x, (x.shape[-1],), self.n1, 1e-5)
        if self.tp > 1:
            h = _AllGatherRows.apply(h, group)
        qkv = TF.linear(h, self.qkv).view(B, S, self.nq + 2 * self.nkv, self.D)
        q, k, v = qkv.split([self.nq, self.nkv, self.nkv], dim=2)

        def rope(t):
            t1, t2 = t[..., : self.D // 2], t[..., self.D // 2:]
            return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1)

        q, k = rope(q), rope(k)
        a = TF.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True)
        a = TF.linear(a.transpose(1, 2).reshape(B * S, self.nq * self.D), self.o)
        if self.tp > 1:
            a = _ReduceScatterRows.apply(a, group)
        x = x + a
        h = TF.rms_norm(x, (x.shape[-1],), self.n2, 1e-5)
        if self.tp > 1:
            h = _AllGatherRows.apply(h, group)
        g, u = TF.linear(h, self.gu).chunk(2, dim=-1)
        m = TF.linear(TF.silu(g) * u, self.down)
        if self.tp > 1:
            m = _ReduceScatterRows.apply(m, group)
        return x + m


def main(args) -> int:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        dist.init_process_group("nccl")
        group = dist.group.WORLD
    H, I, L, nq, nkv, D, V = 4096, 14336, args.layers or 32, 32, 8, 128, 128256
    S, GB, tp = args.seq_len, args.global_batch, world
    torch.manual_seed(1234 + rank)
    layers = torch.nn.ModuleList([Layer(H, I, nq, nkv, D, tp, dev) for _ in range(L)])
    emb = torch.nn.Parameter(torch.randn(V, H, device=dev, dtype=torch.bfloat16) * 0.02)
    head = torch.nn.Parameter(torch.randn(V // tp, H, device=dev, dtype=torch.bfloat16) * 0.02)
    fnorm = torch.nn.Parameter(torch.ones(H, device=dev, dtype=torch.bfloat16))
    params = list(layers.parameters()) + [emb, head, fnorm]
    opt = torch.optim.AdamW(params, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    pos = torch.arange(S, device=dev)[:, None] * (500000.0 ** (-torch.arange(0, D, 2, device=dev) / D))[None]
    cos, sin = pos.cos()[None, :, None, :].bfloat16(), pos.sin()[None, :, None, :].bfloat16()
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, V, (8, S + 1), generator=g).to(dev)

    def micro(i):
        tok = ids[i % 8]
        x = emb[tok[:-1]]
        if tp > 1:
            x = x[rank * (S // tp):(rank + 1) * (S // tp)]
        for l in layers:
            x = l(x, cos, sin, group, 1, S)
        x = TF.rms_norm(x, (H,), fnorm, 1e-5)
        if tp > 1:
            x = _AllGatherRows.apply(x, group)
        loss = 0.0
        labels = tok[1:]
        for c in range(0, S, 2048):                       # chunked head + loss: full logits would be [S, V] fp32
            logits = TF.linear(x[c:c + 2048], head).float()
            if tp > 1:                                    # vocabulary-parallel cross entropy from per-shard statistics
                mx = logits.max(-1, keepdim=True)[0]
                dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
                se = (logits - mx).exp().sum(-1, keepdim=True)
                dist.all_reduce(se, group=group)          # (no gradient through the normaliser's reduction: context arm only)
                lo = rank * (V // tp)
                lab = labels[c:c + 2048] - lo
                ok = (lab >= 0) & (lab < V // tp)
                picked = torch.where(ok, logits.gather(1, lab.clamp(0, V // tp - 1)[:, None])[:, 0], torch.zeros_like(mx[:, 0]))
                loss = loss + ((mx[:, 0] + se[:, 0].log()) / tp - picked).sum()
            else:
                loss = loss + TF.cross_entropy(logits, labels[c:c + 2048], reduction="sum")
        (loss / (S * GB)).backward()

    def step():
        for i in range(GB):
            micro(i)
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)

    W, K = args.warmup, args.steps
    for _ in range(W):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms) / K
    if rank == 0:
        print(json.dumps({"impl": "torch-baseline", "metric": "train_tokens_per_second", "value": GB * S / (ms_per_step / 1e3),
                          "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step, "dtype": "bf16",
                          "config": {"model": "Llama-3-8B", "global_batch": GB, "seq_len": S, "micro_batch": 1, "layers": L,
                                     "parallelism": f"tp{world}" + ("+sp" if world > 1 else ""),
                                     "optimizer": "torch.optim.AdamW(fused), bf16 parameters / gradients / moments",
                                     "note": "stock PyTorch operators (cuBLAS, SDPA, NCCL); context only, not the reference"}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0
