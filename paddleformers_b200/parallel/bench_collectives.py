"""Fused compute + collective kernels against their NCCL + GEMM baseline and their roofline, on the shapes of the
Llama-3-8B tensor-parallel layers:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29520 \
        -m paddleformers_b200.parallel.bench_collectives

For every case prints the device time (CUDA events, max over ranks, L2 flushed between launches) of the fused kernel
and of the baseline, and the fraction of the roofline = max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s) /
measured time.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from ..ops import functional as F
from . import fused_collectives as fc
from .tensor_parallel import all_gather_tokens, reduce_scatter_tokens
from .topology import ParallelDegrees, initialize_parallel

NVLINK_GBS = 770.0


def _peak_tflops():
    for p in ("MEASURED_PEAKS.json",):
        if os.path.exists(p):
            return json.load(open(p))["bf16_tflops"]
    return 1590.0


def _time(fn, iters=10, warmup=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        tot += s.elapsed_time(e)
    t = torch.tensor([tot / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ps = initialize_parallel(ParallelDegrees(mp=int(os.environ["WORLD_SIZE"])))
    tp, rank = ps.degrees.mp, ps.coord["mp"]
    ws = fc.get_tp_workspace()
    group = ps.group("mp")
    T, H, I, QKV = 4096, 4096, 14336, 6144
    peak = _peak_tflops()
    rows = []
    cases = [("qkv  AG->GEMM", "ag", H, QKV // tp, False), ("gate_up AG->GEMM+SwiGLU", "ag", H, 2 * I // tp, True),
             ("o_proj GEMM->RS", "rs", H // tp, H, False), ("down GEMM->RS", "rs", I // tp, H, False)]
    for name, kind, K, N, swiglu in cases:
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        if kind == "ag":
            x = torch.randn(T // tp, K, device="cuda", dtype=torch.bfloat16)
            bufs = ws.layer_gather_buffers(T, K)
            fused = lambda: fc._ag_gemm(ws, bufs, x, w, False, swiglu)
            base = lambda: (F.linear_swiglu if swiglu else F.linear)(all_gather_tokens(x, group), w)
            nv_bytes = (tp - 1) * (T // tp) * K * 2
        else:
            x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
            fused = lambda: fc._gemm_rs(ws, x, w, False)
            base = lambda: reduce_scatter_tokens(F.linear(x, w), group)
            nv_bytes = (tp - 1) * (T // tp) * N * 2
        flops = 2.0 * T * N * K
        t_f, t_b = _time(fused), _time(base)
        roof_ms = max(flops / (peak * 1e12), nv_bytes / (NVLINK_GBS * 1e9)) * 1e3
        rows.append(f"tp{tp} {name:26s} K={K:5d} N={N:5d}: fused {t_f * 1e3:7.1f} us | NCCL+GEMM {t_b * 1e3:7.1f} us | "
                    f"roofline {roof_ms * 1e3:6.1f} us ({'comm' if nv_bytes / (NVLINK_GBS * 1e9) > flops / (peak * 1e12) else 'flops'}-bound) | "
                    f"fused/roofline {roof_ms / t_f:.2f} of measured peaks")
        if rank == 0:
            print(rows[-1], flush=True)
    F.check_kernel_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
