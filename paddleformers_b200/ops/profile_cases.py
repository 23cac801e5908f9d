"""Small fixed workloads of each hot kernel for profiler captures:

    python -m paddleformers_b200.ops.profile_cases --case gemm|attn_fwd|attn_bwd|gemm_swiglu|gemm_wgrad

Each case launches its kernel a few times on inputs larger than the L2 cache but well under a few GB, so that an
``ncu --set full -k regex:<kernel> -c 1`` capture finishes in about a minute.
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


def case_attn(kind: str):
    B, S, Hq, Hkv = 1, 4096, 16, 4
    q = torch.randn(B, S, Hq, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    for _ in range(3):
        out = F.flash_attention(q, k, v, causal=True)
        if kind == "attn_bwd":
            out.backward(torch.ones_like(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=["gemm", "gemm_swiglu", "gemm_wgrad", "attn_fwd", "attn_bwd"])
    args = ap.parse_args()
    if args.case.startswith("gemm"):
        case_gemm(args.case)
    else:
        case_attn(args.case)
    torch.cuda.synchronize()
    F.check_kernel_status()
    print("ok", args.case)


if __name__ == "__main__":
    main()
