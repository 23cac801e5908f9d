"""Quantisation-aware training linears (a8w8 / a8w4 with straight-through estimators) and the Hadamard rotation used
to flatten activation outliers before low-bit quantisation.

Counterparts: ``QATFunc`` and the a8w8 / a8w4 linears of paddleformers/quantization/qat_utils.py:358 and
quantization_linear.py, and the Hadamard utilities of paddleformers/quantization/hadamard_utils.py. The forward pass
sees exactly the values an int8 x int8 (or int8 x int4) kernel would multiply; the backward pass treats the rounding as
identity inside the clipping range.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as TF


class _FakeQuant(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, qmax):
        q = torch.round(x / scale).clamp(-qmax, qmax)
        ctx.save_for_backward((x / scale).abs() <= qmax)
        return q * scale

    @staticmethod
    def backward(ctx, g):
        (inside,) = ctx.saved_tensors
        return g * inside, None, None


def fake_quant_per_token(x: torch.Tensor, bits: int = 8) -> torch.Tensor:
    """Symmetric dynamic quantisation with one scale per token (last dim reduced)."""
    qmax = 2 ** (bits - 1) - 1
    scale = x.detach().abs().amax(-1, keepdim=True).clamp(min=1e-8) / qmax
    return _FakeQuant.apply(x, scale, qmax)


def fake_quant_per_channel(w: torch.Tensor, bits: int = 8) -> torch.Tensor:
    """Symmetric quantisation with one scale per output channel (row of a [out, in] weight)."""
    qmax = 2 ** (bits - 1) - 1
    scale = w.detach().abs().amax(1, keepdim=True).clamp(min=1e-8) / qmax
    return _FakeQuant.apply(w, scale, qmax)


def hadamard_transform(x: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    """Fast Walsh-Hadamard transform along the last dimension (a power of two), O(n log n)."""
    n = x.shape[-1]
    assert n & (n - 1) == 0, "Hadamard transform needs a power-of-two width"
    y = x.reshape(-1, n)
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        y = torch.stack([y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]], dim=2)
        h *= 2
    y = y.reshape(x.shape)
    return y / math.sqrt(n) if normalize else y


def block_hadamard(x: torch.Tensor, block: int) -> torch.Tensor:
    """Hadamard rotation applied independently to consecutive blocks of the last dimension."""
    n = x.shape[-1]
    assert n % block == 0
    return hadamard_transform(x.reshape(*x.shape[:-1], n // block, block)).reshape(x.shape)


class QATLinear(nn.Module):
    """Linear whose forward multiplies fake-quantised activations (per token) by fake-quantised weights (per output
    channel); ``hadamard_block`` > 0 rotates both operands block-wise first, which leaves the product unchanged in exact
    arithmetic and spreads outliers over the block before rounding."""

    def __init__(self, linear: nn.Linear, act_bits: int = 8, weight_bits: int = 8, hadamard_block: int = 0):
        super().__init__()
        self.weight, self.bias = linear.weight, linear.bias
        self.act_bits, self.weight_bits, self.hadamard_block = act_bits, weight_bits, hadamard_block

    def forward(self, x):
        w = self.weight
        if self.hadamard_block:
            x = block_hadamard(x, self.hadamard_block)
            w = block_hadamard(w, self.hadamard_block)
        return TF.linear(fake_quant_per_token(x, self.act_bits), fake_quant_per_channel(w, self.weight_bits), self.bias)


def convert_to_qat(model: nn.Module, algo: str = "a8w8", skip=("lm_head", "gate"), hadamard_block: int = 0) -> int:
    """Replace ``nn.Linear`` modules by ``QATLinear`` sharing their parameters. ``algo``: a8w8 | a8w4."""
    bits = {"a8w8": (8, 8), "a8w4": (8, 4)}[algo]
    n = 0
    for name, mod in list(model.named_modules()):
        if isinstance(mod, nn.Linear) and not any(s in name for s in skip):
            parent_name, _, leaf = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            setattr(parent, leaf, QATLinear(mod, bits[0], bits[1], hadamard_block))
            n += 1
    return n
