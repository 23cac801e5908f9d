"""Kernel micro-benchmarks: ``python -m paddleformers_b200.ops.bench_kernels [--what gemm,attn,elementwise,fp8]``.

Times each kernel with CUDA events on the launching stream after warm-up, flushing L2 between timed launches by
writing a 256 MiB buffer, and prints achieved TFLOP/s or GB/s next to the library kernel of the same shape
(torch.matmul / SDPA) and, when ``MEASURED_PEAKS.json`` sits in the working directory, the fraction of the measured
peak.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import functional as F


def _peaks():
    for p in ("MEASURED_PEAKS.json", os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")):
        if os.path.exists(p):
            with open(p) as f:
                return json.load(f)
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


_flush = None


def timeit(fn, iters=10, warmup=3, flush=True):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters  # ms


def bench_gemm(rows):
    peaks = _peaks()
    shapes = [
        # (name, M, N, K, a_mn, b_mn, epi)
        ("qkv fwd", 4096, 6144, 4096, False, False, F.EPI_STORE_BF16),
        ("o fwd", 4096, 4096, 4096, False, False, F.EPI_STORE_BF16),
        ("gate_up fwd", 4096, 28672, 4096, False, False, F.EPI_STORE_BF16),
        ("gate_up+swiglu", 4096, 28672, 4096, False, False, F.EPI_SWIGLU_BF16),
        ("down fwd", 4096, 4096, 14336, False, False, F.EPI_STORE_BF16),
        ("gate_up dgrad", 4096, 4096, 28672, False, True, F.EPI_STORE_BF16),
        ("down dgrad", 4096, 14336, 4096, False, True, F.EPI_STORE_BF16),
        ("gate_up wgrad", 28672, 4096, 4096, True, True, F.EPI_ACCUM_F32),
        ("down wgrad", 4096, 14336, 4096, True, True, F.EPI_ACCUM_F32),
        ("qkv dgrad", 4096, 4096, 6144, False, True, F.EPI_STORE_BF16),
        ("qkv wgrad", 6144, 4096, 4096, True, True, F.EPI_ACCUM_F32),
        ("o wgrad", 4096, 4096, 4096, True, True, F.EPI_ACCUM_F32),
        ("o_proj 1/8 of K", 4096, 4096, 512, False, False, F.EPI_STORE_BF16),
        ("lm_head 2k", 2048, 128256, 4096, False, False, F.EPI_STORE_BF16),
        ("square 8k", 8192, 8192, 8192, False, False, F.EPI_STORE_BF16),
    ]
    for name, M, N, K, a_mn, b_mn, epi in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
        if epi == F.EPI_ACCUM_F32:
            out = torch.zeros(M, N, device="cuda", dtype=torch.float32)
        elif epi == F.EPI_SWIGLU_BF16:
            out = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        else:
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        res = {}
        for bn in (128, 256, 0):       # 0 = automatic choice: CTA pairs (256 x 256 tiles) on these shapes
            ms = timeit(lambda: F.gemm(a, b, out=out, a_mn=a_mn, b_mn=b_mn, epi=epi, force_bn=bn))
            res[bn] = flops / ms / 1e9
        am = a.t() if a_mn else a
        bm = b if b_mn else b.t()
        ms_lib = timeit(lambda: torch.matmul(am, bm))
        lib = flops / ms_lib / 1e9
        best = max(res.values())
        rows.append(f"gemm {name:16s} M={M} N={N} K={K}: bn128 {res[128]:7.1f} bn256 {res[256]:7.1f} pair {res[0]:7.1f} TFLOP/s | "
                    f"torch.matmul {lib:7.1f} | best/measured-peak {best / peaks['bf16_tflops']:.2f}")
        print(rows[-1], flush=True)
        del a, b, out
    F.check_kernel_status()


def _doc_kend(B, S, lo=128, hi=4096, seed=0):
    g = torch.Generator().manual_seed(seed)
    kend = torch.empty(B, S, dtype=torch.int32)
    for b in range(B):
        pos = 0
        while pos < S:
            end = min(S, pos + int(torch.randint(lo, hi + 1, (1,), generator=g)))
            kend[b, pos:end] = end
            pos = end
    return kend.cuda()


def bench_attn(rows):
    """Forward and backward against torch SDPA on the same line (model FLOPs of the causal half; the packed-document
    case counts the visible (query, key) pairs)."""
    cases = [(1, 4096, 32, 8, False), (1, 4096, 4, 1, False), (2, 4096, 32, 4, True), (1, 8192, 32, 8, False)]
    for (B, S, Hq, Hkv, docs) in cases:
        q = torch.randn(B, S, Hq, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        kend = _doc_kend(B, S) if docs else None
        if docs:
            i = torch.arange(S, device="cuda")
            pairs = float(sum(int(((i[None, :] <= i[:, None]) & (i[:, None] < kend[b][None, :])).sum()) for b in range(B)))
        else:
            pairs = B * S * (S + 1) / 2.0
        flops = 4.0 * Hq * 128 * pairs
        ms = timeit(lambda: F.flash_attention(q, k, v, causal=True, kend=kend))
        out = F.flash_attention(q, k, v, causal=True, kend=kend)
        g = torch.randn_like(out)
        ms_b = timeit(lambda: torch.autograd.grad(out, (q, k, v), g, retain_graph=True), iters=5)
        line = (f"attn B={B} S={S} Hq={Hq} Hkv={Hkv}{' packed docs' if docs else ''}: fwd {flops / ms / 1e9:7.1f} TFLOP/s ({ms * 1e3:.0f} us), "
                f"bwd {2.5 * flops / ms_b / 1e9:7.1f} TFLOP/s ({ms_b * 1e3:.0f} us)")
        if not docs:
            qs, ks, vs = (t.detach().permute(0, 2, 1, 3).requires_grad_() for t in (q, k, v))
            sd = lambda: torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=True)
            ms_lib = timeit(sd)
            o2 = sd()
            g2 = torch.randn_like(o2)
            ms_lib_b = timeit(lambda: torch.autograd.grad(o2, (qs, ks, vs), g2, retain_graph=True), iters=5)
            line += f" | torch SDPA fwd {flops / ms_lib / 1e9:7.1f}, bwd {2.5 * flops / ms_lib_b / 1e9:7.1f}"
        rows.append(line)
        print(line, flush=True)
        del q, k, v, out, g
    F.check_kernel_status()


def bench_elementwise(rows):
    peaks = _peaks()
    T, H, I = 8192, 4096, 14336
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: torch.ops.pfb200.rms_norm_fwd(x, None, w, 1e-5))
    rows.append(f"rms_norm fwd [{T},{H}]: {2 * x.numel() * 2 / ms / 1e6:7.1f} GB/s ({2 * x.numel() * 2 / ms / 1e6 / peaks['hbm_gbs']:.2f} of measured copy)")
    print(rows[-1], flush=True)
    # backward: reads dy, x and the residual-stream gradient, writes dx; the weight-gradient partials are folded by a second kernel
    ops = torch.ops.pfb200
    rstd = torch.ones(T, device="cuda")
    dwf = torch.zeros(H, device="cuda")
    scratch = torch.empty(int(ops.rms_norm_bwd_scratch_rows()) * H, device="cuda")
    ms = timeit(lambda: ops.rms_norm_bwd(x, x, w, rstd, x, dwf, True, scratch))
    rows.append(f"rms_norm bwd [{T},{H}] (+residual grad, dw): {4 * x.numel() * 2 / ms / 1e6:7.1f} GB/s "
                f"({4 * x.numel() * 2 / ms / 1e6 / peaks['hbm_gbs']:.2f} of measured copy)")
    print(rows[-1], flush=True)
    # rotary embedding in place on the q and k heads of a packed qkv activation (32 + 8 heads of 128 in rows of 6144)
    qkv = torch.randn(T, 6144, device="cuda", dtype=torch.bfloat16)
    cos, sin = F.rope_tables(T, 128, 500000.0, qkv.device)
    ms = timeit(lambda: ops.rope_inplace(qkv, None, cos, sin, 40, 128, 128, False))
    rows.append(f"rope in place [{T}, 40 heads x 128]: {2 * T * 40 * 128 * 2 / ms / 1e6:7.1f} GB/s "
                f"({2 * T * 40 * 128 * 2 / ms / 1e6 / peaks['hbm_gbs']:.2f} of measured copy)")
    print(rows[-1], flush=True)
    # per-head RMSNorm + rotary on 32 heads of 128 (Qwen3), forward and backward
    xq = torch.randn(T, 32 * 128, device="cuda", dtype=torch.bfloat16)
    nw = torch.ones(128, device="cuda", dtype=torch.bfloat16)
    oq = torch.empty_like(xq)
    ms = timeit(lambda: ops.qk_norm_rope_fwd(xq, oq, nw, None, cos, sin, 32, 128, 128, 1e-6))
    rstd_q = ops.qk_norm_rope_fwd(xq, oq, nw, None, cos, sin, 32, 128, 128, 1e-6)
    dnw = torch.zeros(128, device="cuda")
    ms_b = timeit(lambda: ops.qk_norm_rope_bwd(oq, xq, nw, rstd_q, xq.new_empty(xq.shape), dnw, None, cos, sin, 32, 128, 128))
    rows.append(f"qk_norm + rope [{T}, 32 heads x 128]: forward {2 * xq.numel() * 2 / ms / 1e6:7.1f} GB/s, backward "
                f"{3 * xq.numel() * 2 / ms_b / 1e6:7.1f} GB/s ({3 * xq.numel() * 2 / ms_b / 1e6 / peaks['hbm_gbs']:.2f} of measured copy)")
    print(rows[-1], flush=True)
    gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: torch.ops.pfb200.swiglu_fwd(gu))
    rows.append(f"swiglu fwd [{T},{2 * I}]: {3 * T * I * 2 / ms / 1e6:7.1f} GB/s")
    print(rows[-1], flush=True)
    n = 1 << 28
    p, m, v, g = (torch.zeros(n, device="cuda") for _ in range(4))
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    sc = torch.tensor([1e-3, 1.0, 0.1, 0.05, 0.0], device="cuda")
    ms = timeit(lambda: torch.ops.pfb200.adamw_step(p, m, v, g, p16, sc, 0.9, 0.95, 1e-8, 0.1), flush=False)
    rows.append(f"adamw {n} elems: {n * 30 / ms / 1e6:7.1f} GB/s ({n * 30 / ms / 1e6 / peaks['hbm_gbs']:.2f} of measured copy)")
    print(rows[-1], flush=True)
    logits = torch.randn(2048, 128256, device="cuda", dtype=torch.bfloat16)
    labels = torch.randint(0, 128256, (2048,), device="cuda")
    loss = torch.empty(2048, device="cuda")
    d = torch.empty(1, device="cuda")
    one = torch.ones(1, device="cuda")
    ms = timeit(lambda: torch.ops.pfb200.cross_entropy(logits, labels, loss, d, d, d, one, 0, -100, 0, True))
    rows.append(f"cross_entropy [2048,128256]: {ms:.3f} ms, {logits.numel() * 2 * 2 / ms / 1e6:7.1f} GB/s (read+write once)")
    print(rows[-1], flush=True)


def bench_fp8(rows):
    """Block-scaled e4m3 GEMM and its quantisation kernels; beside them the bf16 tcgen05 GEMM of the same shape and
    ``torch._scaled_mm`` with the same 1x128 / 128x128 scales where this torch build offers it."""
    from ..quantization import fp8 as Q

    for name, M, N, K in (("dsv3 gate_up", 4096, 4096, 7168), ("dsv3 down", 4096, 7168, 2048), ("square", 8192, 8192, 8192)):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        xq, xs_t = Q.quant_act_kernel(x)
        wq, ws = Q.quant_weight_kernel(w)
        ops = torch.ops.pfb200
        bn = int(ops.mxf8_tile_n(N))
        sfa = ops.mx_pack_scales(xs_t, True, M, 1, 128)
        sfb = ops.mx_pack_scales(ws, False, N, 1, bn)
        ms = timeit(lambda: ops.gemm_mxf8(xq, sfa, wq, sfb, out, None, 0, bn))          # scales applied by the tensor core
        ms_promo = timeit(lambda: Q.fp8_gemm(xq, xs_t, wq, ws, out=out, pow2=False))      # scales applied in the epilogue
        ms_pack = timeit(lambda: ops.mx_pack_scales(xs_t, True, M, 1, 128))
        ms_bf16 = timeit(lambda: F.gemm(x, w, out=out))
        ms_qa = timeit(lambda: Q.quant_act_kernel(x))
        ms_qw = timeit(lambda: Q.quant_weight_kernel(w))
        ms_qt = timeit(lambda: Q.quant_transpose_kernel(x))
        acc = torch.zeros(N, K, device="cuda")
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        ms_wg = timeit(lambda: Q.fp8_wgrad(dy, x, acc))                                   # two transposing quantisers + packs + GEMM
        ms_wg_bf16 = timeit(lambda: F.gemm(dy, x, out=acc, a_mn=True, b_mn=True, epi=F.EPI_ACCUM_F32))
        fl = 2.0 * M * N * K
        lib = float("nan")
        try:
            xs = xs_t.t().contiguous()
            lib_ms = timeit(lambda: torch._scaled_mm(xq, wq.t(), scale_a=xs, scale_b=ws.t(), out_dtype=torch.bfloat16))
            lib = fl / lib_ms / 1e9
        except Exception:  # this torch build has no 1x128 / 128x128 scaled matmul
            pass
        rows.append(f"fp8 gemm {name:13s} M={M} N={N} K={K} tile {bn}: {fl / ms / 1e9:7.1f} TFLOP/s tensor-core scaling "
                    f"(epilogue promotion {fl / ms_promo / 1e9:7.1f}, bf16 kernel {fl / ms_bf16 / 1e9:7.1f}, torch._scaled_mm {lib:7.1f}) | "
                    f"scale pack {ms_pack * 1e3:5.1f} us | wgrad fp8 end to end {fl / ms_wg / 1e9:7.1f} vs bf16 {fl / ms_wg_bf16 / 1e9:7.1f} TFLOP/s | "
                    f"quant act {x.numel() * 3 / ms_qa / 1e6:6.0f} GB/s, quant transpose {x.numel() * 3 / ms_qt / 1e6:6.0f} GB/s, "
                    f"quant weight {w.numel() * 3 / ms_qw / 1e6:6.0f} GB/s")
        print(rows[-1], flush=True)
    # fused SwiGLU + quantisation against SwiGLU then quantisation (rows x 2I -> e4m3 rows x I)
    R, I = 16384, 2048
    gu = torch.randn(R, 2 * I, device="cuda", dtype=torch.bfloat16)
    dact = torch.randn(R, I, device="cuda", dtype=torch.bfloat16)
    ops = torch.ops.pfb200
    ms_f = timeit(lambda: ops.swiglu_quant_fwd(gu, None, True, False))
    ms_u = timeit(lambda: Q.quant_act_kernel(ops.swiglu_fwd(gu)))
    ms_fb = timeit(lambda: ops.swiglu_quant_bwd(dact, gu, None, True, True))
    ms_ub = timeit(lambda: Q.quant_act_kernel(ops.swiglu_bwd(dact, gu, True)[0]))
    rows.append(f"swiglu+quant [{R}, 2x{I}]: forward fused {ms_f * 1e3:6.1f} us ({R * I * 5 / ms_f / 1e6:5.0f} GB/s) vs two kernels {ms_u * 1e3:6.1f} us; "
                f"backward fused {ms_fb * 1e3:6.1f} us ({R * I * 14 / ms_fb / 1e6:5.0f} GB/s) vs two kernels {ms_ub * 1e3:6.1f} us")
    print(rows[-1], flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,attn,elementwise")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    F._ops()                 # load the extension before the first torch.ops.pfb200 lookup
    rows = []
    for w in args.what.split(","):
        {"gemm": bench_gemm, "attn": bench_attn, "elementwise": bench_elementwise, "fp8": bench_fp8}[w](rows)
    if args.out:
        with open(args.out, "w") as f:
            f.write("\n".join(rows) + "\n")


if __name__ == "__main__":
    main()
