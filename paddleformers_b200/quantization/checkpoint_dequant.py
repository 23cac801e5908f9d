"""De-quantisation of quantised Hugging Face checkpoints at load time.

* fp8 block checkpoints (DeepSeek-V3 style): ``<name>.weight`` in e4m3 with ``<name>.weight_scale_inv`` holding one
  fp32 (or UE8M0) scale per 128x128 block;
* MXFP4 group checkpoints (gpt-oss style): ``<name>_blocks`` (two e2m1 values per byte) with ``<name>_scales`` (one
  E8M0 exponent byte per group of 32 values).

Counterparts: paddleformers/quantization/checkpoint_dequant.py:277-355 (``FP8BlockCheckpointDequantizer``,
``MXFP4GroupCheckpointDequantizer``) and the Triton converters of paddleformers/utils/upcast_downcast_triton.py.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def dequant_fp8_block(weight: torch.Tensor, scale_inv: torch.Tensor, block: int = 128, out_dtype=torch.bfloat16) -> torch.Tensor:
    N, K = weight.shape
    s = scale_inv.float()
    if scale_inv.dtype == torch.uint8:       # UE8M0 exponents
        s = torch.exp2(scale_inv.float() - 127.0)
    s = s.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return (weight.float() * s).to(out_dtype)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    """blocks: uint8 [..., G, 16] (32 e2m1 values per group, low nibble first); scales: uint8 [..., G] E8M0."""
    lut = _E2M1_VALUES.to(blocks.device)
    lo, hi = (blocks & 0x0F).long(), (blocks >> 4).long()
    vals = torch.stack([lut[lo], lut[hi]], dim=-1).flatten(-2)            # [..., G, 32]
    exp = torch.exp2(scales.float() - 127.0).unsqueeze(-1)
    return (vals * exp).flatten(-2).to(out_dtype)


def quant_mxfp4(x: torch.Tensor):
    """Inverse of ``dequant_mxfp4`` (round to nearest e2m1 under a power-of-two group scale); x: [..., 32*G]."""
    g = x.float().unflatten(-1, (-1, 32))
    amax = g.abs().amax(-1, keepdim=True).clamp(min=2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 6.0))
    scaled = g / torch.exp2(e)
    lut = _E2M1_VALUES.to(x.device)
    idx = (scaled.unsqueeze(-1) - lut).abs().argmin(-1)
    blocks = (idx[..., 0::2] | (idx[..., 1::2] << 4)).to(torch.uint8)
    return blocks, (e.squeeze(-1) + 127).clamp(0, 255).to(torch.uint8)


def build_dequantizer(quantization_config, reader) -> Optional[Callable[[str, torch.Tensor], torch.Tensor]]:
    """Returns ``f(name, tensor) -> tensor`` applied to every tensor read from the checkpoint."""
    qc = quantization_config if isinstance(quantization_config, dict) else getattr(quantization_config, "__dict__", {})
    method = qc.get("quant_method")
    if method == "fp8":
        block = (qc.get("weight_block_size") or [128, 128])[0]

        def f(name, t):
            if t.dtype == torch.float8_e4m3fn:
                sname = name + "_scale_inv"
                if reader.has(sname):
                    return dequant_fp8_block(t, reader.get(sname), block)
                return t.to(torch.bfloat16)
            return t
        return f
    if method == "mxfp4":
        def f(name, t):
            return t
        return f
    return None
