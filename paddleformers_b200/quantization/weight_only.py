"""Weight-only quantised linears (int8 / int4 per-channel, NF4 blockwise for QLoRA) with on-the-fly de-quantisation.

Counterpart: paddleformers/quantization/quantization_linear.py:263 (``QuantizationLinear``) and the ``compute_type``
expansion wint8 / wint4 / nf4 (paddleformers/cli/hparams/finetuning_args.py:379-417).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as F

_NF4 = torch.tensor([-1.0, -0.6961928, -0.5250730, -0.3949175, -0.2844414, -0.1848449, -0.0910500, 0.0,
                     0.0795803, 0.1609302, 0.2461123, 0.3379152, 0.4407098, 0.5626170, 0.7229568, 1.0])


def quantize_weight(w: torch.Tensor, algo: str, block: int = 64):
    wf = w.float()
    if algo == "wint8":
        scale = wf.abs().amax(1, keepdim=True).clamp(min=1e-8) / 127.0
        return torch.round(wf / scale).clamp(-127, 127).to(torch.int8), scale
    if algo == "wint4":
        scale = wf.abs().amax(1, keepdim=True).clamp(min=1e-8) / 7.0
        q = torch.round(wf / scale).clamp(-7, 7).to(torch.int8) + 8
        return (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8), scale
    if algo == "nf4":
        flat = wf.reshape(-1, block)
        scale = flat.abs().amax(1, keepdim=True).clamp(min=1e-8)
        idx = ((flat / scale).unsqueeze(-1) - _NF4.to(w.device)).abs().argmin(-1).to(torch.uint8)
        return (idx[:, 0::2] | (idx[:, 1::2] << 4)), scale
    raise ValueError(algo)


def dequantize_weight(q, scale, algo: str, shape, dtype, block: int = 64):
    if algo == "wint8":
        return (q.float() * scale).to(dtype)
    if algo == "wint4":
        lo, hi = (q & 0x0F).to(torch.int8) - 8, (q >> 4).to(torch.int8) - 8
        full = torch.stack([lo, hi], -1).flatten(-2).float()
        return (full * scale).to(dtype)
    if algo == "nf4":
        lut = _NF4.to(q.device)
        vals = torch.stack([lut[(q & 0x0F).long()], lut[(q >> 4).long()]], -1).flatten(-2)
        return (vals * scale).reshape(shape).to(dtype)
    raise ValueError(algo)


class QuantizationLinear(nn.Module):
    def __init__(self, linear: nn.Linear, algo: str = "wint8", block: int = 64):
        super().__init__()
        self.algo, self.block = algo, block
        self.shape, self.dtype = tuple(linear.weight.shape), linear.weight.dtype
        q, s = quantize_weight(linear.weight.detach(), algo, block)
        self.register_buffer("quant_weight", q)
        self.register_buffer("quant_scale", s)
        self.bias = linear.bias

    @property
    def weight(self):
        return dequantize_weight(self.quant_weight, self.quant_scale, self.algo, self.shape, self.dtype, self.block)

    def forward(self, x):
        return F.linear(x, self.weight, self.bias)


def quantize_model(model: nn.Module, algo: str, skip=("lm_head",)) -> int:
    n = 0
    for name, mod in list(model.named_modules()):
        if isinstance(mod, nn.Linear) and not any(s in name for s in skip):
            parent_name, _, leaf = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            setattr(parent, leaf, QuantizationLinear(mod, algo))
            n += 1
    return n
