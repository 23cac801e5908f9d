"""Block-scaled fp8 (e4m3) quantisation: 1x128 activation blocks, 128x128 weight blocks, fp32 or power-of-two (UE8M0)
scales; reference math for the CUDA quantisation kernels and the fp8 linear layers.

Counterparts: paddleformers/transformers/fp8_utils.py:105-131, 262-268 (block shapes), the Triton
``act_quant_kernel`` / ``weight_dequant_kernel`` (paddleformers/cli/train/deepseek_v3_pretrain/kernel.py:29-125) and
the UE8M0 flag (paddleformers/transformers/configuration_utils.py:454-459).
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.nn as nn

FP8_MAX = 448.0
BLOCK = 128


def _pow2_scale(s: torch.Tensor) -> torch.Tensor:
    """Round scales up to the next power of two (the value an UE8M0 byte can hold)."""
    return torch.exp2(torch.ceil(torch.log2(s.clamp(min=2.0 ** -127))))


def quant_act_1x128(x: torch.Tensor, ue8m0: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """x: [T, K] -> (e4m3 [T, K], scales fp32 [T, ceil(K/128)]) with x ~= q * scale per 1x128 block."""
    T, K = x.shape
    nb = (K + BLOCK - 1) // BLOCK
    pad = nb * BLOCK - K
    xf = torch.nn.functional.pad(x.float(), (0, pad)).view(T, nb, BLOCK)
    amax = xf.abs().amax(-1).clamp(min=1e-12)
    scale = amax / FP8_MAX
    if ue8m0:
        scale = _pow2_scale(scale)
    q = (xf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).view(T, nb * BLOCK)[:, :K].to(torch.float8_e4m3fn)
    return q, scale


def quant_weight_128x128(w: torch.Tensor, ue8m0: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """w: [N, K] -> (e4m3 [N, K], scales fp32 [ceil(N/128), ceil(K/128)])."""
    N, K = w.shape
    nn_, nk = (N + BLOCK - 1) // BLOCK, (K + BLOCK - 1) // BLOCK
    wf = torch.nn.functional.pad(w.float(), (0, nk * BLOCK - K, 0, nn_ * BLOCK - N)).view(nn_, BLOCK, nk, BLOCK)
    amax = wf.abs().amax(dim=(1, 3)).clamp(min=1e-12)
    scale = amax / FP8_MAX
    if ue8m0:
        scale = _pow2_scale(scale)
    q = (wf / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(nn_ * BLOCK, nk * BLOCK)[:N, :K].to(torch.float8_e4m3fn)
    return q, scale


def dequant_act(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    T, K = q.shape
    s = scale.repeat_interleave(BLOCK, dim=1)[:, :K]
    return q.float() * s


def dequant_weight(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    s = scale.repeat_interleave(BLOCK, dim=0)[:N].repeat_interleave(BLOCK, dim=1)[:, :K]
    return q.float() * s


def _use_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


def quant_act_kernel(x: torch.Tensor, ue8m0: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """CUDA 1x128 quantisation of a bf16 [T, K] tensor (K % 128 == 0): (e4m3 [T, K], scales fp32 TRANSPOSED
    [K/128, T], the layout the fp8 GEMM epilogue reads with coalesced loads)."""
    from ..ops import functional as F

    return F._ops().fp8_quant_act(x.contiguous(), ue8m0)


def quant_weight_kernel(w: torch.Tensor, ue8m0: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """CUDA 128x128 quantisation of a bf16 [N, K] weight (K % 128 == 0): (e4m3 [N, K], scales fp32 [ceil(N/128), K/128])."""
    from ..ops import functional as F

    return F._ops().fp8_quant_weight(w.contiguous(), ue8m0)


def _mx_enabled() -> bool:
    return os.environ.get("PFB_FP8_MX", "1") != "0"


def _packed_weight_scales(ws: torch.Tensor, rows_per_group: int, groups: int, bn: int) -> torch.Tensor:
    """Exponent words of a 128x128-scaled weight for ``bn``-row tiles, cached on the scale tensor (weight caches are
    rebuilt, as new tensors, after every optimizer step)."""
    cache = getattr(ws, "_mx_pack", None)
    if cache is None:
        cache = {}
        ws._mx_pack = cache
    key = (rows_per_group, groups, bn)
    if key not in cache:
        cache[key] = torch.ops.pfb200.mx_pack_scales(ws, False, rows_per_group, groups, bn)
    return cache[key]


def fp8_gemm(xq, xs_t, wq, ws, block_expert=None, n_per_expert: int = 0, out=None, pow2: bool = True) -> torch.Tensor:
    """Block-scaled e4m3 product on the tcgen05 tensor cores: out[M, N] (bf16) = dequant(xq, xs_t^T) @ dequant(wq, ws)^T.
    With ``block_expert`` (int32, one entry per 128 rows of xq, -1 = skip) ``wq`` holds E stacked [n_per_expert, K]
    matrices and each row block is multiplied by its expert's matrix.

    ``pow2`` says that every scale is a power of two (the UE8M0 option of the quantisers): the product then runs on the
    tensor core's own block scaling (``gemm_mxf8``); otherwise the partial sums are promoted in the epilogue
    (``gemm_fp8``). ``PFB_FP8_MX=0`` forces the latter."""
    from ..ops import functional as F

    ops = F._ops()
    M, K = xq.shape
    grouped = block_expert is not None
    N = n_per_expert if grouped else wq.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
    if pow2 and _mx_enabled() and M > 0:
        bn = int(ops.mxf8_tile_n(N))
        groups = wq.shape[0] // N if grouped else 1
        sfa = ops.mx_pack_scales(xs_t, True, M, 1, 128)
        sfb = _packed_weight_scales(ws, N, groups, bn)
        ops.gemm_mxf8(xq, sfa, wq, sfb, out, block_expert, n_per_expert, bn)
    else:
        ops.gemm_fp8(xq, xs_t, wq, ws, out, block_expert, n_per_expert)
    return out


def quant_transpose_kernel(x: torch.Tensor, ue8m0: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """CUDA transposing quantisation of a bf16 [T, K] tensor: (e4m3 [K, ceil(T/128)*128] = x^T with a zero tail,
    scales fp32 [ceil(T/128), K]), one scale per channel and 128 tokens."""
    return torch.ops.pfb200.fp8_quant_transpose(x if x.stride(1) == 1 else x.contiguous(), ue8m0)


def fp8_wgrad(dy: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Weight gradient dy^T @ x ([N, K] fp32) with both operands in e4m3, scaled per 128 tokens, on the tensor core's
    block scaling; ADDED to ``out`` when given (an fp32 main-grad buffer), returned as a new fp32 tensor otherwise
    (the fp8 wgrad of paddleformers/transformers/fp8_utils.py:1011-1190)."""
    from ..ops import functional as F

    ops = F._ops()
    N, K = dy.shape[1], x.shape[1]
    aq, as_ = quant_transpose_kernel(dy)
    bq, bs = quant_transpose_kernel(x)
    bn = int(ops.mxf8_tile_n(K))
    sfa = ops.mx_pack_scales(as_, True, N, 1, 128)
    sfb = ops.mx_pack_scales(bs, True, K, 1, bn)
    if out is None:
        out = torch.zeros((N, K), dtype=torch.float32, device=dy.device)
    ops.gemm_mxf8(aq, sfa, bq, sfb, out, None, 0, bn)
    return out


def fp8_gemm_reference(xq, xs, wq, ws) -> torch.Tensor:
    """Block-scaled product x @ w^T in fp32: per 128-wide K block, partial products are scaled by
    act_scale[t, kb] * weight_scale[n // 128, kb] (the math of the reference's Triton fp8 GEMM,
    paddleformers/cli/train/deepseek_v3_pretrain/kernel.py:129-186)."""
    return dequant_act(xq, xs) @ dequant_weight(wq, ws).t()


def _fp8_wgrad_ok(dy2: torch.Tensor, x2: torch.Tensor) -> bool:
    """The fp8 weight gradient needs power-of-two scales, channel counts that the transposing quantiser tiles (64) and is
    switched by PFB_FP8_WGRAD (default on)."""
    return (os.environ.get("PFB_FP8_WGRAD", "1") != "0" and _mx_enabled() and dy2.shape[1] % 64 == 0 and x2.shape[1] % 64 == 0
            and dy2.shape[0] >= 128)


class _FP8LinearFn(torch.autograd.Function):
    """fp8 forward, input-gradient and weight-gradient products with bf16 master weights. The forward and input-gradient
    operands are scaled per 1x128 block along their contraction (channels); the weight gradient contracts over tokens,
    so both of its operands are quantised again, transposed, with one scale per channel and 128 tokens."""

    @staticmethod
    def forward(ctx, x, weight, wq, ws, wq_t, ws_t, ue8m0):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.kernels = _use_kernels(x2) and wq_t is not None
        if ctx.kernels:
            xq, xs_t = quant_act_kernel(x2, ue8m0)
            y = fp8_gemm(xq, xs_t, wq, ws, pow2=ue8m0)
        else:
            xq, xs = quant_act_1x128(x2, ue8m0)
            y = fp8_gemm_reference(xq, xs, wq, ws).to(x.dtype)
        ctx.save_for_backward(x2, weight, wq, ws, wq_t if wq_t is not None else wq, ws_t if ws_t is not None else ws)
        ctx.ue8m0, ctx.shape = ue8m0, x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight, wq, ws, wq_t, ws_t = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if ctx.kernels:
            from ..ops import functional as F

            dq, ds_t = quant_act_kernel(dy2, ctx.ue8m0)
            dx = fp8_gemm(dq, ds_t, wq_t, ws_t, pow2=ctx.ue8m0).view(ctx.shape)   # dy @ W with the transposed fp8 weight copy
            if _fp8_wgrad_ok(dy2, x2):
                mg = getattr(weight, "main_grad", None)
                dw = fp8_wgrad(dy2, x2, mg.view(weight.shape) if mg is not None else None)
                dw = None if mg is not None else dw.to(weight.dtype)
            else:
                dw = F._weight_grad(dy2.contiguous(), x2, weight)     # bf16 tcgen05 wgrad (into main_grad when present)
            return dx, dw, None, None, None, None, None
        dq, ds = quant_act_1x128(dy2, ctx.ue8m0)
        dx = (dequant_act(dq, ds) @ dequant_weight(wq, ws)).to(dy.dtype).view(ctx.shape)
        mg = getattr(weight, "main_grad", None)
        dw = dy2.float().t() @ x2.float()
        if mg is not None:
            mg.add_(dw)
            return dx, None, None, None, None, None, None
        return dx, dw.to(weight.dtype), None, None, None, None, None


class FP8Linear(nn.Module):
    """Linear layer computing in block-scaled fp8 with a cached quantised copy of the bf16 master weight; the cache is
    refreshed after each optimizer step by ``FP8QuantWeightCallback``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, ue8m0: bool = True, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.ue8m0 = ue8m0
        self._wq = self._ws = self._wq_t = self._ws_t = None
        nn.init.normal_(self.weight, std=0.02)

    def refresh_fp8_weight_cache(self):
        """Quantise the bf16 master weight (and, on the GPU, its transpose for the input-gradient product)."""
        with torch.no_grad():
            w = self.weight.detach()
            if _use_kernels(w) and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
                self._wq, self._ws = quant_weight_kernel(w, self.ue8m0)
                self._wq_t, self._ws_t = quant_weight_kernel(w.t().contiguous(), self.ue8m0)
            else:
                self._wq, self._ws = quant_weight_128x128(w, self.ue8m0)
                self._wq_t = self._ws_t = None

    def forward(self, x):
        if self._wq is None or self._wq.device != self.weight.device:
            self.refresh_fp8_weight_cache()
        y = _FP8LinearFn.apply(x, self.weight, self._wq, self._ws, self._wq_t, self._ws_t, self.ue8m0)
        return y + self.bias if self.bias is not None else y


def convert_linears_to_fp8(model: nn.Module, skip=("lm_head", "gate")) -> int:
    """Replace ``nn.Linear`` modules by ``FP8Linear`` sharing the same parameters; returns the number converted."""
    n = 0
    for name, mod in list(model.named_modules()):
        # the GEMM kernels tile both weight dimensions by 128 (the forward product and its transposed copy for the input
        # gradient); other layers (e.g. DeepSeek's 576-wide compressed key/value projection) stay in bf16
        if isinstance(mod, nn.Linear) and not any(s in name for s in skip) and mod.in_features % 128 == 0 \
                and mod.out_features % 128 == 0:
            parent_name, _, leaf = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            new = FP8Linear(mod.in_features, mod.out_features, mod.bias is not None, dtype=mod.weight.dtype, device=mod.weight.device)
            new.weight = mod.weight
            new.bias = mod.bias
            setattr(parent, leaf, new)
            n += 1
    return n
