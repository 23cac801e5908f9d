"""Functional operators of the framework.

Every operator has two implementations that compute the same thing:

* CUDA tensors run the hand-written sm_100a kernels of the in-tree extension (``torch.ops.pfb200.*``). There is no
  silent fallback: if the extension is not built the call raises.
* CPU tensors (tests, gloo ranks, tiny configs) run a plain PyTorch implementation in the tensor's own dtype.

The autograd wrappers implement the "main_grad" convention of the reference's mixed-precision trainer
(``amp_master_grad`` / ``fused_linear_param_grad_add``, paddleformers/trainer/training_args.py:2143): when a weight
has a ``main_grad`` attribute (fp32, same shape) the weight-gradient GEMM accumulates straight into it and autograd
sees no ``.grad`` for that parameter.
"""
from __future__ import annotations

import os

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _build

EPI_STORE_BF16, EPI_STORE_F32, EPI_ACCUM_F32, EPI_SWIGLU_BF16, EPI_ACCUM_BF16 = 0, 1, 2, 3, 4

_scratch = {}


def _ops():
    if not _build.load_extension(required=True):  # pragma: no cover - raises inside
        raise RuntimeError("pfb200 extension unavailable")
    return torch.ops.pfb200


def use_cuda_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda


def _get_scratch(device, numel: int) -> torch.Tensor:
    """Persistent fp32 scratch buffer per device (block partials of reductions); grows on demand."""
    key = (device.type, device.index)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(max(numel, 1 << 20), dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


def check_kernel_status(reset: bool = True) -> int:
    """Synchronise and return the device status word (0 = ok); raises on a recorded kernel error."""
    code = int(_ops().read_status(reset))
    if code != 0:
        raise RuntimeError(f"pfb200 kernel reported error status {code} (bounded wait expired or bounds check failed)")
    return code


_replayed_launches = 0


def add_replayed_launches(n: int) -> None:
    """Kernels launched by replaying a captured CUDA graph never pass through the host-side launchers; the owner of
    the graph reports how many of this library's kernels one replay contains."""
    global _replayed_launches
    _replayed_launches += int(n)


def kernel_launch_count(reset: bool = False) -> int:
    """Number of this library's kernels launched so far (eager launches + kernels inside replayed graphs)."""
    global _replayed_launches
    if not _build.is_loaded() and not _build.load_extension():
        return 0
    n = int(torch.ops.pfb200.launch_count(reset)) + _replayed_launches
    if reset:
        _replayed_launches = 0
    return n


# ----------------------------------------------------------------------------------------------------------------
# GEMM
# ----------------------------------------------------------------------------------------------------------------
def gemm(a, b, out=None, *, a_mn=False, b_mn=False, epi=EPI_STORE_BF16, out2=None, block_expert=None,
         n_per_expert=0, force_bn=0):
    """D = A @ B^T on the tcgen05 kernel. ``a``: [M,K] or (a_mn) [K,M]; ``b``: [N,K] or (b_mn) [K,N]."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = n_per_expert if block_expert is not None else (b.shape[1] if b_mn else b.shape[0])
    if out is None:
        n_out = N // 2 if epi == EPI_SWIGLU_BF16 else N
        dt = torch.float32 if epi in (EPI_STORE_F32, EPI_ACCUM_F32) else torch.bfloat16
        out = torch.empty((M, n_out), dtype=dt, device=a.device)
    _ops().gemm(a, b, out, a_mn, b_mn, epi, out2, block_expert, n_per_expert, force_bn)
    return out


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.x_shape = x.shape
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16 != 0:
            x2 = x2.contiguous()
        # allocate the result in its final shape: returning a view made inside the Function would forbid later
        # in-place ops (rotary embedding) on it
        y = torch.empty((*x.shape[:-1], weight.shape[0]), dtype=x.dtype, device=x.device)
        gemm(x2, weight, out=y.view(-1, weight.shape[0]))
        if bias is not None:
            y += bias
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1 or (dy2.stride(0) * dy2.element_size()) % 16 != 0:
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = _weight_grad(dy2, x2, weight)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0)
        return dx, dw, db


def split_bf16(t: torch.Tensor):
    """t (fp32) ~= hi + lo with both parts in bf16: 16 mantissa bits survive instead of 8, and products of a bf16
    operand with (hi, lo) accumulated in fp32 on the tensor cores reproduce an fp32 matmul to ~1e-5 relative."""
    hi = t.to(torch.bfloat16)
    lo = (t - hi.float()).to(torch.bfloat16)
    return hi, lo


class _RouterLogitsFn(torch.autograd.Function):
    """fp32-accurate router logits x @ W^T for bf16 activations and fp32 router weights on the tcgen05 GEMM: the weight
    (and, in the backward pass, the logit gradient) is split into bf16 hi + lo parts that ride along as extra rows /
    columns of one GEMM each, so no fp32 copy of the activations is made and no CUDA-core GEMM runs."""

    @staticmethod
    def forward(ctx, x, w):
        E = w.shape[0]
        hi, lo = split_bf16(w.detach())
        out = gemm(x, torch.cat([hi, lo], 0), epi=EPI_STORE_F32)          # [T, 2E]
        ctx.save_for_backward(x, hi, lo)
        return out[:, :E] + out[:, E:]

    @staticmethod
    def backward(ctx, g):
        x, hi, lo = ctx.saved_tensors
        E = hi.shape[0]
        ghi, glo = split_bf16(g.float())
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # (g_hi + g_lo) @ (W_hi + W_lo), dropping the lo x lo term
            dx = gemm(torch.cat([ghi, glo, ghi], 1), torch.cat([hi, hi, lo], 0), b_mn=True)
        if ctx.needs_input_grad[1]:
            both = gemm(torch.cat([ghi, glo], 1), x, a_mn=True, b_mn=True, epi=EPI_STORE_F32)   # [2E, H]
            dw = both[:E] + both[E:]
        return dx, dw


def router_logits(x2d: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Router scores in fp32 ([T, E]) from activations [T, H] and fp32 weights [E, H]
    (paddleformers/nn/moe_deepep/moe_gate.py:464-499 computes them with an fp32 matmul)."""
    if (use_cuda_kernels(x2d) and x2d.dtype == torch.bfloat16 and weight.dtype == torch.float32 and weight.shape[0] % 8 == 0
            and weight.shape[1] % 8 == 0 and x2d.is_contiguous()):
        return _RouterLogitsFn.apply(x2d, weight)
    return torch.nn.functional.linear(x2d.float(), weight.float())


class WeightGradStore:
    """Queue of deferred weight-gradient GEMMs, for pipeline schedules that run the input-gradient part of a backward
    pass (which the previous stage is waiting for) before its weight-gradient part. While a group is open, linear
    layers whose weights accumulate into ``main_grad`` enqueue their dW GEMM instead of launching it; the schedule runs
    the group later. Only such layers can be deferred: their dW is not a value autograd has to return."""

    _open = None
    _groups: list = []

    @classmethod
    def begin_group(cls):
        cls._open = []

    @classmethod
    def end_group(cls):
        if cls._open is not None:
            cls._groups.append(cls._open)
        cls._open = None

    @classmethod
    def defer(cls, fn) -> bool:
        if cls._open is None:
            return False
        cls._open.append(fn)
        return True

    @classmethod
    def run_group(cls):
        if cls._groups:
            for fn in cls._groups.pop(0):
                fn()

    @classmethod
    def run_all(cls):
        while cls._groups:
            cls.run_group()


def _weight_grad(dy2, x2, weight):
    """dW = dy^T x. Accumulates into ``weight.main_grad`` (fp32) when present and returns None for autograd."""
    mg = getattr(weight, "main_grad", None)
    if mg is not None and WeightGradStore.defer(
            lambda: gemm(dy2, x2, out=mg.view(weight.shape), a_mn=True, b_mn=True, epi=EPI_ACCUM_F32)):
        return None
    if mg is not None:
        gemm(dy2, x2, out=mg.view(weight.shape), a_mn=True, b_mn=True, epi=EPI_ACCUM_F32)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True, epi=EPI_STORE_BF16)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ weight^T (+ bias); weight is [out, in] (the Hugging Face / torch layout)."""
    if use_cuda_kernels(x) and x.dtype == torch.bfloat16:
        return _LinearFn.apply(x, weight, bias)
    return F.linear(x, weight, bias)


class _LinearSwigluFn(torch.autograd.Function):
    """act = silu(x Wg^T) * (x Wu^T) with W = [Wg; Wu] stacked on rows; SwiGLU runs in the GEMM epilogue and the
    raw gate|up projection is kept for the backward pass."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.x_shape = x.shape
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        T, N = x2.shape[0], weight.shape[0]
        raw = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
        act = torch.empty((*x.shape[:-1], N // 2), dtype=torch.bfloat16, device=x.device)
        gemm(x2, weight, out=act.view(-1, N // 2), epi=EPI_SWIGLU_BF16, out2=raw)
        ctx.save_for_backward(x2, weight, raw)
        return act

    @staticmethod
    def backward(ctx, dact):
        x2, weight, raw = ctx.saved_tensors
        d2 = dact.reshape(-1, dact.shape[-1]).contiguous()
        dgu, _ = _ops().swiglu_bwd(d2, raw, False)
        dx = gemm(dgu, weight, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(dgu, x2, weight) if ctx.needs_input_grad[1] else None
        return dx, dw


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Fused gate/up projection + SwiGLU. ``weight`` = [gate rows; up rows] = [2*I, H]."""
    if use_cuda_kernels(x) and x.dtype == torch.bfloat16:
        return _LinearSwigluFn.apply(x, weight)
    gu = F.linear(x, weight)
    g, u = gu.chunk(2, dim=-1)
    return F.silu(g) * u


# ----------------------------------------------------------------------------------------------------------------
# RMSNorm / SwiGLU
# ----------------------------------------------------------------------------------------------------------------
def _rms_norm_ref(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        r2 = residual.reshape(-1, shape[-1]).contiguous() if residual is not None else None
        y, rstd, s = _ops().rms_norm_fwd(x2, r2, w, eps)
        ctx.save_for_backward(s if residual is not None else x2.contiguous(), w, rstd)
        ctx.has_res = residual is not None
        ctx.shape = shape
        if residual is not None:
            return y.view(shape), s.view(shape)
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy, dsum=None):
        x2, w, rstd = ctx.saved_tensors
        H = x2.shape[-1]
        dy2 = dy.reshape(-1, H)
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        ops = _ops()
        scratch = _get_scratch(x2.device, int(ops.rms_norm_bwd_scratch_rows()) * H)
        mg = getattr(w, "main_grad", None)
        dres = dsum.reshape(-1, H).contiguous() if (ctx.has_res and dsum is not None) else None
        if mg is not None:
            dx = ops.rms_norm_bwd(dy2, x2, w, rstd, dres, mg, True, scratch)
            dw = None
        else:
            dwf = torch.empty(H, dtype=torch.float32, device=x2.device)
            dx = ops.rms_norm_bwd(dy2, x2, w, rstd, dres, dwf, False, scratch)
            dw = dwf.to(w.dtype)
        dx = dx.view(ctx.shape)
        if ctx.has_res:
            return dx, dw, None, dx
        return dx, dw, None, None


def rms_norm(x, weight, eps: float = 1e-6, residual: Optional[torch.Tensor] = None):
    """RMSNorm over the last dim. With ``residual`` returns (norm(x + residual), x + residual)."""
    if use_cuda_kernels(x) and x.dtype == torch.bfloat16:
        return _RmsNormFn.apply(x, weight, eps, residual)
    if residual is not None:
        s = x + residual
        return _rms_norm_ref(s, weight, eps), s
    return _rms_norm_ref(x, weight, eps)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        shape = gu.shape
        g2 = gu.reshape(-1, shape[-1])
        if g2.stride(-1) != 1:
            g2 = g2.contiguous()
        ctx.save_for_backward(g2)
        ctx.shape = shape
        return _ops().swiglu_fwd(g2).view(*shape[:-1], shape[-1] // 2)

    @staticmethod
    def backward(ctx, dact):
        (g2,) = ctx.saved_tensors
        dgu, _ = _ops().swiglu_bwd(dact.reshape(-1, dact.shape[-1]).contiguous(), g2, False)
        return dgu.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up with gate = first half, up = second half of the last dim."""
    if use_cuda_kernels(gate_up) and gate_up.dtype == torch.bfloat16:
        return _SwigluFn.apply(gate_up)
    g, u = gate_up.chunk(2, dim=-1)
    return F.silu(g) * u


# ----------------------------------------------------------------------------------------------------------------
# Rotary embedding (+ per-head QK RMSNorm)
# ----------------------------------------------------------------------------------------------------------------
def rope_uses_long_factors(scaling: Optional[dict], seq_len: int) -> bool:
    """'longrope' keeps two sets of per-frequency factors; the long set applies once the sequence exceeds the original
    context length."""
    if not scaling or scaling.get("rope_type", scaling.get("type")) not in ("longrope", "su"):
        return False
    return int(seq_len) > int(scaling.get("original_max_position_embeddings", 0) or 0)


def rope_tables(positions_max: int, rot_dim: int, theta: float, device, scaling: Optional[dict] = None,
                seq_len: Optional[int] = None, max_position_embeddings: Optional[int] = None):
    """fp32 cos/sin tables [positions_max, rot_dim/2]; supports the 'llama3', 'linear', 'yarn', 'longrope' and 'dynamic'
    scaling rules of paddleformers/transformers/modeling_rope_utils.py. ``seq_len`` (default: the table length) is the
    sequence length the rules that depend on it see: 'longrope' switches to its long factors beyond the original context,
    'dynamic' grows the base beyond ``max_position_embeddings``."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    attn_factor = 1.0
    cur = int(seq_len or positions_max)
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type", "default"))
        factor = float(scaling.get("factor", 1.0))
        if kind in ("longrope", "su"):
            orig = int(scaling.get("original_max_position_embeddings", 0) or max_position_embeddings or positions_max)
            ext = scaling["long_factor"] if cur > orig else scaling["short_factor"]
            inv_freq = inv_freq / torch.tensor(ext, dtype=torch.float64)
            full = float(max_position_embeddings or orig)
            ratio = float(scaling["factor"]) if scaling.get("factor") else full / orig
            attn_factor = float(scaling.get("attention_factor") or
                                (1.0 if ratio <= 1.0 else math.sqrt(1.0 + math.log(ratio) / math.log(orig))))
        elif kind == "dynamic":
            mp = int(max_position_embeddings or scaling.get("original_max_position_embeddings") or positions_max)
            if cur > mp:
                base = theta * ((factor * cur / mp) - (factor - 1)) ** (rot_dim / (rot_dim - 2))
                inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
        elif kind == "linear":
            inv_freq = inv_freq / factor
        elif kind == "llama3":
            low = float(scaling.get("low_freq_factor", 1.0))
            high = float(scaling.get("high_freq_factor", 4.0))
            old = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = (old / wavelen - low) / (high - low)
            scaled = torch.where(wavelen > old / low, inv_freq / factor, inv_freq)
            mid = (wavelen <= old / low) & (wavelen >= old / high)
            inv_freq = torch.where(mid, (1 - smooth) * inv_freq / factor + smooth * inv_freq, scaled)
        elif kind == "yarn":
            old = float(scaling.get("original_max_position_embeddings", 4096))
            beta_fast = float(scaling.get("beta_fast", 32))
            beta_slow = float(scaling.get("beta_slow", 1))

            def corr_dim(n_rot):
                return (rot_dim * math.log(old / (n_rot * 2 * math.pi))) / (2 * math.log(theta))

            lo, hi = corr_dim(beta_fast), corr_dim(beta_slow)
            if scaling.get("truncate", True):          # some families keep the fractional correction range
                lo, hi = math.floor(lo), math.ceil(hi)
            lo, hi = max(lo, 0), min(hi, rot_dim - 1)
            ramp = ((torch.arange(rot_dim // 2, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
            mask = 1 - ramp
            inv_freq = inv_freq / factor * (1 - mask) + inv_freq * mask
            mscale = float(scaling.get("mscale", 1.0))
            mscale_all = float(scaling.get("mscale_all_dim", 0.0))

            def get_mscale(s, m):
                return 1.0 if s <= 1 else 0.1 * m * math.log(s) + 1.0

            attn_factor = get_mscale(factor, mscale) / get_mscale(factor, mscale_all) if mscale_all else get_mscale(factor, mscale)
    t = torch.arange(positions_max, dtype=torch.float64)
    freqs = torch.outer(t, inv_freq)
    return (freqs.cos() * attn_factor).float().to(device), (freqs.sin() * attn_factor).float().to(device)


def _rope_ref(x, cos, sin, positions, rot):
    # x: [T, nh, D]; cos/sin: [P, rot/2]
    c = cos[positions] if positions is not None else cos[: x.shape[0]]
    s = sin[positions] if positions is not None else sin[: x.shape[0]]
    c = c[:, None, :].to(torch.float32)
    s = s[:, None, :].to(torch.float32)
    xf = x.float()
    x1, x2, rest = xf[..., : rot // 2], xf[..., rot // 2: rot], xf[..., rot:]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)
    return out.to(x.dtype)


class _RopeFn(torch.autograd.Function):
    """Rotates q and k in place inside one fused [T, (hq + 2 hkv) * D] buffer (or any 2-D strided view)."""

    @staticmethod
    def forward(ctx, x, cos, sin, positions, n_heads, D, rot):
        ctx.mark_dirty(x)
        _ops().rope_inplace(x, positions, cos, sin, n_heads, D, rot, False)
        ctx.save_for_backward(cos, sin, positions if positions is not None else torch.empty(0))
        ctx.meta = (n_heads, D, rot, positions is not None)
        return x

    @staticmethod
    def backward(ctx, dx):
        cos, sin, pos = ctx.saved_tensors
        n_heads, D, rot, has_pos = ctx.meta
        dx = dx.contiguous() if dx.stride(-1) != 1 else dx.clone()
        _ops().rope_inplace(dx, pos if has_pos else None, cos, sin, n_heads, D, rot, True)
        return dx, None, None, None, None, None, None


def rope_heads(x2d: torch.Tensor, cos, sin, positions, n_heads: int, head_dim: int, rot_dim: Optional[int] = None):
    """Rotary embedding on the first ``n_heads`` heads of a [T, >= n_heads*head_dim] tensor (half-rotation layout:
    first and second half of the rotated dims pair up). Out of place on CPU; on CUDA rotates a fresh copy in place."""
    rot = rot_dim or head_dim
    if use_cuda_kernels(x2d) and x2d.dtype == torch.bfloat16:
        pos32 = positions.to(torch.int32) if positions is not None else None
        return _RopeFn.apply(x2d.clone(), cos, sin, pos32, n_heads, head_dim, rot)
    T = x2d.shape[0]
    head = x2d[:, : n_heads * head_dim].reshape(T, n_heads, head_dim)
    out = _rope_ref(head, cos, sin, positions, rot).reshape(T, n_heads * head_dim)
    if x2d.shape[1] > n_heads * head_dim:
        out = torch.cat([out, x2d[:, n_heads * head_dim:]], dim=-1)
    return out


class _QkNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, nw, cos, sin, positions, n_heads, D, rot, eps):
        out = torch.empty((x.shape[0], n_heads * D), dtype=x.dtype, device=x.device)
        rstd = _ops().qk_norm_rope_fwd(x, out, nw, positions, cos, sin, n_heads, D, rot, eps)
        ctx.save_for_backward(x, nw, rstd, cos, sin, positions if positions is not None else torch.empty(0))
        ctx.meta = (n_heads, D, rot, positions is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, nw, rstd, cos, sin, pos = ctx.saved_tensors
        n_heads, D, rot, has_pos = ctx.meta
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        dx = torch.empty((x.shape[0], n_heads * D), dtype=x.dtype, device=x.device)
        mg = getattr(nw, "main_grad", None)
        dnw = mg if mg is not None else torch.zeros(D, dtype=torch.float32, device=x.device)
        _ops().qk_norm_rope_bwd(dout, x, nw, rstd, dx, dnw, pos if has_pos else None, cos, sin, n_heads, D, rot)
        return dx, (None if mg is not None else dnw.to(nw.dtype)), None, None, None, None, None, None, None


def qk_norm_rope(x2d, norm_weight, cos, sin, positions, n_heads: int, head_dim: int, rot_dim: Optional[int] = None,
                 eps: float = 1e-6):
    """Per-head RMSNorm over head_dim followed by rotary embedding (Qwen3 / GLM-4.5 QK-norm). x2d: [T, n_heads*D]
    (row-strided views of a fused qkv buffer are fine)."""
    rot = rot_dim or head_dim
    if use_cuda_kernels(x2d) and x2d.dtype == torch.bfloat16:
        pos32 = positions.to(torch.int32) if positions is not None else None
        return _QkNormRopeFn.apply(x2d, norm_weight, cos, sin, pos32, n_heads, head_dim, rot, eps)
    T = x2d.shape[0]
    h = x2d.reshape(T, n_heads, head_dim)
    h = _rms_norm_ref(h, norm_weight, eps)
    return _rope_ref(h, cos, sin, positions, rot).reshape(T, n_heads * head_dim)


# ----------------------------------------------------------------------------------------------------------------
# Embedding
# ----------------------------------------------------------------------------------------------------------------
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, vocab_start):
        ctx.save_for_backward(ids, weight)
        ctx.vocab_start = vocab_start
        return _ops().embedding_fwd(ids.reshape(-1), weight, vocab_start).view(*ids.shape, weight.shape[1])

    @staticmethod
    def backward(ctx, dout):
        ids, weight = ctx.saved_tensors
        mg = getattr(weight, "main_grad", None)
        d2 = dout.reshape(-1, dout.shape[-1]).contiguous()
        if mg is not None:
            _ops().embedding_bwd(ids.reshape(-1), d2, mg.view(weight.shape), ctx.vocab_start)
            return None, None, None
        g = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        _ops().embedding_bwd(ids.reshape(-1), d2, g, ctx.vocab_start)
        return None, g.to(weight.dtype), None


def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Row gather; ids outside [vocab_start, vocab_start + rows) give zero rows (vocabulary-parallel shards)."""
    if use_cuda_kernels(weight) and weight.dtype == torch.bfloat16:
        return _EmbeddingFn.apply(ids, weight, vocab_start)
    local = ids - vocab_start
    ok = (local >= 0) & (local < weight.shape[0])
    out = F.embedding(local.clamp(0, weight.shape[0] - 1), weight)
    return out * ok.unsqueeze(-1).to(out.dtype)


# ----------------------------------------------------------------------------------------------------------------
# Attention
# ----------------------------------------------------------------------------------------------------------------
def dense_mask_from_kend(kend: Optional[torch.Tensor], S: int, causal: bool, device) -> torch.Tensor:
    """Boolean [B or 1, S, S] visibility mask (True = attend) from FlashMask-style start rows: key column j is
    masked for rows i >= kend[b, j]; causal additionally masks j > i
    (paddleformers/utils/masking_utils.py:69-113)."""
    i = torch.arange(S, device=device)[:, None]
    j = torch.arange(S, device=device)[None, :]
    vis = (j <= i) if causal else torch.ones(S, S, dtype=torch.bool, device=device)
    vis = vis[None]
    if kend is not None:
        vis = vis & (i[None] < kend[:, None, :].to(device))
    return vis


def attention_reference(q, k, v, causal=True, kend=None, scale=None):
    """Plain PyTorch attention in fp32. q: [B,S,Hq,D], k/v: [B,S,Hkv,D(v)]."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    vis = dense_mask_from_kend(kend, S, causal, q.device)[:, None]
    s = s.masked_fill(~vis, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)


# "deterministic": dQ contributions of the key tiles are added in a fixed order (bit-identical runs);
# "bwd_heads_per_cta": 0 = chosen from the grid size, 1 = one CTA per query head, 2 = one CTA per KV head (walks its group)
_attn_backend = {"bwd": "auto", "p_in_tmem": True, "deterministic": os.environ.get("PFB_ATTN_DETERMINISTIC", "0") == "1",
                 "bwd_heads_per_cta": 0}


def set_attention_options(**kw):
    _attn_backend.update(kw)


def _kend_tiles(kend: torch.Tensor, S: int):
    B = kend.shape[0]
    tiles = (S + 127) // 128
    pad = tiles * 128 - S
    big = torch.iinfo(torch.int32).max
    kmin = F.pad(kend, (0, pad), value=big).view(B, tiles, 128).amin(-1).to(torch.int32).contiguous()
    kmax = F.pad(kend, (0, pad), value=0).view(B, tiles, 128).amax(-1).to(torch.int32).contiguous()
    return kmin, kmax


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, kend, scale):
        B, S, Hq, D = q.shape
        Hkv = k.shape[2]
        Dv = v.shape[-1]
        q3, k3, v3 = q.reshape(B * S, Hq, D), k.reshape(B * S, Hkv, D), v.reshape(B * S, Hkv, Dv)
        out = torch.empty((B * S, Hq, Dv), dtype=q.dtype, device=q.device)
        kmin = kmax = None
        if kend is not None:
            kend = kend.to(torch.int32).contiguous()
            kmin, kmax = _kend_tiles(kend, S)
        lse = _ops().attn_fwd(q3, k3, v3, out, B, S, scale, causal, kend, kmin, kmax, _attn_backend["p_in_tmem"])
        ctx.save_for_backward(q, k, v, out, lse, kend if kend is not None else torch.empty(0), kmin if kmin is not None else torch.empty(0), kmax if kmax is not None else torch.empty(0))
        ctx.meta = (causal, scale, kend is not None)
        return out.view(B, S, Hq, Dv)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, kend, kmin, kmax = ctx.saved_tensors
        causal, scale, has_kend = ctx.meta
        from . import attention_bwd

        dq, dk, dv = attention_bwd.flash_attention_backward(
            dout, q, k, v, out, lse, causal, kend if has_kend else None, kmin if has_kend else None,
            kmax if has_kend else None, scale)
        return dq, dk, dv, None, None, None


def flash_attention(q, k, v, causal: bool = True, kend: Optional[torch.Tensor] = None, scale: Optional[float] = None):
    """Attention over [B, S, H, D] tensors with GQA, causal and document masks (``kend``: int [B, S], key column j is
    visible to query rows i with j <= i < kend[b, j])."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    # 128-wide heads, or multi-head latent attention (192-wide queries / keys with as many key heads as query heads)
    if use_cuda_kernels(q) and q.dtype == torch.bfloat16 and v.shape[-1] == 128 and (
            D == 128 or (D == 192 and q.shape[2] == k.shape[2] and os.environ.get("PFB_MLA_KERNEL", "1") != "0")):
        return _FlashAttnFn.apply(q, k, v, causal, kend, scale)
    if use_cuda_kernels(q) and q.dtype == torch.bfloat16:
        from . import attention_bwd

        return attention_bwd.attention_generic(q, k, v, causal, kend, scale)
    return attention_reference(q, k, v, causal, kend, scale)


# ----------------------------------------------------------------------------------------------------------------
# Fused lm_head + cross entropy
# ----------------------------------------------------------------------------------------------------------------
class _LinearCrossEntropyFn(torch.autograd.Function):
    """Chunked head GEMM + softmax cross entropy that never materialises the full [T, V] logits: for every chunk of
    rows the logits are produced in bf16, turned into scale * (softmax - onehot) in place and immediately contracted
    into dh and dW, like the reference's FusedHeadAndCrossEntropy
    (paddleformers/transformers/tensor_parallel_utils.py:133-569) which also computes gradients in the forward."""

    @staticmethod
    def forward(ctx, h, weight, labels, ignore_index, chunk, scale, need_grad):
        ops = _ops()
        T, H = h.shape
        V = weight.shape[0]
        dev = h.device
        loss_rows = torch.empty(T, dtype=torch.float32, device=dev)
        dummy = torch.empty(1, dtype=torch.float32, device=dev)
        dh = torch.empty_like(h) if need_grad else None
        mg = getattr(weight, "main_grad", None)
        dw = None
        if need_grad and mg is None:
            dw = torch.zeros((V, H), dtype=torch.float32, device=dev)
        wg = mg.view(V, H) if mg is not None else dw
        sc = scale.reshape(1).to(torch.float32)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            hc = h[s:e]
            logits = gemm(hc, weight)
            ops.cross_entropy(logits, labels[s:e], loss_rows[s:e], dummy, dummy, dummy, sc, 0, ignore_index, 0, need_grad)
            if need_grad:
                gemm(logits, weight, out=dh[s:e], b_mn=True)
                gemm(logits, hc, out=wg, a_mn=True, b_mn=True, epi=EPI_ACCUM_F32)
        ctx.save_for_backward(dh if need_grad else torch.empty(0), dw if dw is not None else torch.empty(0))
        ctx.has_dw = dw is not None
        ctx.wdtype = weight.dtype
        count = (labels != ignore_index).sum()
        ctx.mark_non_differentiable(count)
        return loss_rows.sum() * sc[0], count

    @staticmethod
    def backward(ctx, dloss, _dcount):
        dh, dw = ctx.saved_tensors
        # Gradients already include `scale`. dloss is 1 when the loss is the root of the graph; it is honoured for dh
        # and for a non-main_grad dW (a main_grad weight gradient has already been accumulated).
        return dh * dloss.to(dh.dtype), (dw * dloss).to(ctx.wdtype) if ctx.has_dw else None, None, None, None, None, None


def fused_linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                               chunk: int = 2048, loss_scale: Optional[torch.Tensor] = None):
    """Returns (scaled sum of token losses, number of non-ignored tokens) of softmax-CE(h @ weight^T, labels).

    ``loss_scale``: optional scalar tensor multiplied into the loss *before* gradients are formed (folds the
    1/num_tokens and 1/accumulation factors into the in-forward gradient computation)."""
    h2 = h.reshape(-1, h.shape[-1])
    lab = labels.reshape(-1)
    if use_cuda_kernels(h2) and h2.dtype == torch.bfloat16:
        scale = loss_scale if loss_scale is not None else torch.ones((), dtype=torch.float32, device=h2.device)
        need_grad = torch.is_grad_enabled() and (h2.requires_grad or weight.requires_grad)
        return _LinearCrossEntropyFn.apply(h2.contiguous(), weight, lab.contiguous(), ignore_index, chunk, scale, need_grad)
    logits = F.linear(h2, weight).float()
    loss = F.cross_entropy(logits, lab, ignore_index=ignore_index, reduction="sum")
    cnt = (lab != ignore_index).sum()
    if loss_scale is not None:
        loss = loss * loss_scale
    return loss, cnt


# ----------------------------------------------------------------------------------------------------------------
# Packed-qkv attention (no slicing in autograd: one gradient buffer for q, k and v)
# ----------------------------------------------------------------------------------------------------------------
def _packed_views(qkv2d, B, S, Hq, Hkv, D):
    T = B * S
    q = qkv2d[:, : Hq * D].view(T, Hq, D)
    k = qkv2d[:, Hq * D: (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv2d[:, (Hq + Hkv) * D: (Hq + 2 * Hkv) * D].view(T, Hkv, D)
    return q, k, v


class _FlashAttnPackedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv2d, B, S, Hq, Hkv, D, causal, kend, scale):
        q, k, v = _packed_views(qkv2d, B, S, Hq, Hkv, D)
        out = torch.empty((B * S, Hq, D), dtype=qkv2d.dtype, device=qkv2d.device)
        kmin = kmax = None
        if kend is not None:
            kend = kend.to(torch.int32).contiguous()
            kmin, kmax = _kend_tiles(kend, S)
        lse = _ops().attn_fwd(q, k, v, out, B, S, scale, causal, kend, kmin, kmax, _attn_backend["p_in_tmem"])
        e = torch.empty(0)
        ctx.save_for_backward(qkv2d, out, lse, kend if kend is not None else e, kmin if kmin is not None else e,
                              kmax if kmax is not None else e)
        ctx.meta = (B, S, Hq, Hkv, D, causal, scale, kend is not None)
        return out.view(B * S, Hq * D)

    @staticmethod
    def backward(ctx, dout):
        qkv2d, out, lse, kend, kmin, kmax = ctx.saved_tensors
        B, S, Hq, Hkv, D, causal, scale, has_kend = ctx.meta
        from . import attention_bwd

        q, k, v = _packed_views(qkv2d, B, S, Hq, Hkv, D)
        dqkv = torch.empty_like(qkv2d)
        dq, dk, dv = _packed_views(dqkv, B, S, Hq, Hkv, D)
        attention_bwd.flash_attention_backward_into(
            dout.reshape(B, S, Hq, D), q.view(B, S, Hq, D), k.view(B, S, Hkv, D), v.view(B, S, Hkv, D),
            out.view(B, S, Hq, D), lse, causal, kend if has_kend else None, kmin if has_kend else None,
            kmax if has_kend else None, scale, dq.view(B, S, Hq, D), dk.view(B, S, Hkv, D), dv.view(B, S, Hkv, D))
        return dqkv, None, None, None, None, None, None, None, None


def flash_attention_qkvpacked(qkv2d, B: int, S: int, Hq: int, Hkv: int, D: int, causal: bool = True,
                              kend: Optional[torch.Tensor] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Attention on a fused [B*S, (Hq + 2*Hkv) * D] projection (q heads | k heads | v heads). Returns [B*S, Hq*D]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if use_cuda_kernels(qkv2d) and qkv2d.dtype == torch.bfloat16 and D == 128:
        return _FlashAttnPackedFn.apply(qkv2d, B, S, Hq, Hkv, D, causal, kend, scale)
    q, k, v = _packed_views(qkv2d, B, S, Hq, Hkv, D)
    out = flash_attention(q.reshape(B, S, Hq, D), k.reshape(B, S, Hkv, D), v.reshape(B, S, Hkv, D), causal, kend, scale)
    return out.reshape(B * S, Hq * D)


class _QkNormRopePackedFn(torch.autograd.Function):
    """qkv -> new packed buffer with q and k per-head RMS-normalised and rotated, v copied."""

    @staticmethod
    def forward(ctx, qkv2d, qw, kw, cos, sin, positions, Hq, Hkv, D, rot, eps):
        ops = _ops()
        out = torch.empty_like(qkv2d)
        qi, ki = qkv2d[:, : Hq * D], qkv2d[:, Hq * D: (Hq + Hkv) * D]
        qo, ko = out[:, : Hq * D], out[:, Hq * D: (Hq + Hkv) * D]
        rq = ops.qk_norm_rope_fwd(qi, qo, qw, positions, cos, sin, Hq, D, rot, eps)
        rk = ops.qk_norm_rope_fwd(ki, ko, kw, positions, cos, sin, Hkv, D, rot, eps)
        out[:, (Hq + Hkv) * D:].copy_(qkv2d[:, (Hq + Hkv) * D:])
        ctx.save_for_backward(qkv2d, qw, kw, rq, rk, cos, sin, positions if positions is not None else torch.empty(0))
        ctx.meta = (Hq, Hkv, D, rot, positions is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv2d, qw, kw, rq, rk, cos, sin, pos = ctx.saved_tensors
        Hq, Hkv, D, rot, has_pos = ctx.meta
        ops = _ops()
        pos = pos if has_pos else None
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        dx = torch.empty_like(qkv2d)
        outs = []
        for (lo, hi, nh, w, r) in ((0, Hq * D, Hq, qw, rq), (Hq * D, (Hq + Hkv) * D, Hkv, kw, rk)):
            mg = getattr(w, "main_grad", None)
            dnw = mg if mg is not None else torch.zeros(D, dtype=torch.float32, device=dx.device)
            ops.qk_norm_rope_bwd(dout[:, lo:hi], qkv2d[:, lo:hi], w, r, dx[:, lo:hi], dnw, pos, cos, sin, nh, D, rot)
            outs.append(None if mg is not None else dnw.to(w.dtype))
        dx[:, (Hq + Hkv) * D:].copy_(dout[:, (Hq + Hkv) * D:])
        return dx, outs[0], outs[1], None, None, None, None, None, None, None, None


def qk_norm_rope_packed(qkv2d, q_norm_w, k_norm_w, cos, sin, positions, Hq, Hkv, D, rot_dim=None, eps=1e-6):
    """Per-head RMSNorm + rotary on the q and k heads of a packed qkv projection; v passes through."""
    rot = rot_dim or D
    if use_cuda_kernels(qkv2d) and qkv2d.dtype == torch.bfloat16:
        pos32 = positions.to(torch.int32) if positions is not None else None
        return _QkNormRopePackedFn.apply(qkv2d, q_norm_w, k_norm_w, cos, sin, pos32, Hq, Hkv, D, rot, eps)
    q = qk_norm_rope(qkv2d[:, : Hq * D], q_norm_w, cos, sin, positions, Hq, D, rot, eps)
    k = qk_norm_rope(qkv2d[:, Hq * D: (Hq + Hkv) * D], k_norm_w, cos, sin, positions, Hkv, D, rot, eps)
    return torch.cat([q, k, qkv2d[:, (Hq + Hkv) * D:]], dim=-1)


def rope_packed(qkv2d, cos, sin, positions, Hq, Hkv, D, rot_dim=None):
    """Rotary embedding on the q and k heads of a packed qkv projection, in place on CUDA (the producing GEMM does
    not need its output for its own backward)."""
    rot = rot_dim or D
    if use_cuda_kernels(qkv2d) and qkv2d.dtype == torch.bfloat16:
        pos32 = positions.to(torch.int32) if positions is not None else None
        return _RopeFn.apply(qkv2d, cos, sin, pos32, Hq + Hkv, D, rot)
    return rope_heads(qkv2d, cos, sin, positions, Hq + Hkv, D, rot)
