"""Small fixed workloads of each hot kernel for profiler captures:

    python -m paddleformers_b200.ops.profile_cases --case gemm|attn_fwd|attn_bwd|gemm_swiglu|gemm_wgrad|gemm_mxf8|moe_layer|moe_layer_local

Each case launches its kernel a few times on inputs larger than the L2 cache but well under a few GB, so that an
``ncu --set full --clock-control none -k regex:<kernel> -s 1 -c 1`` capture finishes in about a minute (always pass
``--clock-control none``: without it the profiler locks the GPU clocks, which other users of a shared machine inherit).
"""
from __future__ import annotations

import argparse

import torch

from . import functional as F


def case_gemm(kind: str):
    M, N, K = 4096, 8192, 4096
    if kind == "gemm":
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            F.gemm(a, b, out=out)
    elif kind == "gemm_swiglu":
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        raw = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            F.gemm(a, b, out=out, epi=F.EPI_SWIGLU_BF16, out2=raw)
    else:  # wgrad: dW[N, K] += dy[T, N]^T x[T, K]
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        out = torch.zeros(N, K, device="cuda", dtype=torch.float32)
        for _ in range(3):
            F.gemm(dy, x, out=out, a_mn=True, b_mn=True, epi=F.EPI_ACCUM_F32)


def case_gemm_mxf8():
    """Block-scaled e4m3 product with the scales applied by the tensor core (kernel gemm_mxf8_kernel)."""
    from ..quantization import fp8 as Q

    M, N, K = 4096, 8192, 4096
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    xq, xs_t = Q.quant_act_kernel(x)
    wq, ws = Q.quant_weight_kernel(w)
    for _ in range(3):
        Q.fp8_gemm(xq, xs_t, wq, ws, out=out)


def case_attn(kind: str):
    B, S, Hq, Hkv = 1, 4096, 16, 4
    q = torch.randn(B, S, Hq, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    for _ in range(3):
        out = F.flash_attention(q, k, v, causal=True)
        if kind == "attn_bwd":
            out.backward(torch.ones_like(out))


def case_moe_layer(kind: str):
    """One MoE layer forward + backward with the per-rank shape of Qwen3-30B-A3B under 8-way expert parallelism
    (16 local experts, 4096 tokens x top-8, hidden 2048, expert width 768). ``moe_layer`` exchanges tokens through the
    peer-memory dispatch / combine kernels (a one-rank group: the rank exchanges with itself), ``moe_layer_local``
    through the local permutation."""
    from ..models.configuration import Qwen3MoeConfig
    from ..nn.moe import MoELayer
    from ..parallel import fused_ep
    from ..parallel.topology import get_parallel_state

    cfg = Qwen3MoeConfig(hidden_size=2048, num_experts=16, num_experts_per_tok=8, moe_intermediate_size=768, intermediate_size=768,
                         num_hidden_layers=1, num_attention_heads=16, num_key_value_heads=4, vocab_size=128)
    layer = MoELayer(cfg, dtype=torch.bfloat16, device="cuda")
    for p in layer.parameters():
        torch.nn.init.normal_(p, std=0.02)
    x = torch.randn(4096, 2048, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn_like(x)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for it in range(4):
        if it == 3:
            start.record()
        if kind == "moe_layer":
            idx, w, _ = layer.gate(x)
            ws = fused_ep.get_workspace(get_parallel_state(), x, layer)
            y = fused_ep.moe_forward(ws, layer, x, idx, w)
        else:
            y = layer(x)
        y.backward(g)
    end.record()
    torch.cuda.synchronize()
    print(f"{kind}: forward+backward {start.elapsed_time(end):.3f} ms")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=["gemm", "gemm_swiglu", "gemm_wgrad", "gemm_mxf8", "attn_fwd", "attn_bwd",
                                                      "moe_layer", "moe_layer_local"])
    args = ap.parse_args()
    if args.case.startswith("moe"):
        case_moe_layer(args.case)
    elif args.case == "gemm_mxf8":
        case_gemm_mxf8()
    elif args.case.startswith("gemm"):
        case_gemm(args.case)
    else:
        case_attn(args.case)
    torch.cuda.synchronize()
    F.check_kernel_status()
    print("ok", args.case)


if __name__ == "__main__":
    main()
