"""De-quantisation of quantised Hugging Face checkpoints at load time.

* fp8 block checkpoints (DeepSeek-V3 style): ``<name>.weight`` in e4m3 with ``<name>.weight_scale_inv`` holding one
  fp32 (or UE8M0) scale per 128x128 block;
* MXFP4 group checkpoints (gpt-oss style): ``<name>_blocks`` (two e2m1 values per byte) with ``<name>_scales`` (one
  E8M0 exponent byte per group of 32 values).

Counterparts: paddleformers/quantization/checkpoint_dequant.py:277-355 (``FP8BlockCheckpointDequantizer``,
``MXFP4GroupCheckpointDequantizer``) and the Triton converters of paddleformers/utils/upcast_downcast_triton.py
(``downcast_to_mxfp`` / ``upcast_from_mxfp`` below). Tensors in host memory go through the compiled, multi-threaded
converters of the host library when it has been built; the tensor-op implementations are the specification and the
fallback (and serve tensors on a device).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


_host = None


def _host_lib():
    """ctypes handle of the host converters (None when the library is not built)."""
    global _host
    if _host is None:
        from ..ops._build import load_host_library

        lib = load_host_library()
        _host = lib if lib is not None and hasattr(lib, "pfb_mxfp4_dequant_bf16") else False
    return _host or None


def _ptr(t: torch.Tensor):
    import ctypes

    return ctypes.c_void_p(t.data_ptr())


def _on_host(*ts) -> bool:
    return all(t.device.type == "cpu" for t in ts) and _host_lib() is not None


def dequant_fp8_block(weight: torch.Tensor, scale_inv: torch.Tensor, block: int = 128, out_dtype=torch.bfloat16,
                      native: bool = True) -> torch.Tensor:
    N, K = weight.shape
    if native and scale_inv.dtype == torch.float32 and weight.dtype == torch.float8_e4m3fn and _on_host(weight, scale_inv):
        import ctypes

        w, sc = weight.contiguous().view(torch.uint8), scale_inv.contiguous()
        out = torch.empty(N, K, dtype=torch.bfloat16)
        _host_lib().pfb_fp8_block_dequant_bf16(_ptr(w), _ptr(sc), _ptr(out), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int64(block))
        return out.to(out_dtype)
    s = scale_inv.float()
    if scale_inv.dtype == torch.uint8:       # UE8M0 exponents
        s = torch.exp2(scale_inv.float() - 127.0)
    s = s.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return (weight.float() * s).to(out_dtype)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, out_dtype=torch.bfloat16, native: bool = True) -> torch.Tensor:
    """blocks: uint8 [..., G, 16] (32 e2m1 values per group, low nibble first); scales: uint8 [..., G] E8M0."""
    if native and _on_host(blocks, scales):
        import ctypes

        b, sc = blocks.contiguous(), scales.contiguous()
        out = torch.empty(tuple(sc.shape[:-1]) + (sc.shape[-1] * 32,), dtype=torch.bfloat16)
        _host_lib().pfb_mxfp4_dequant_bf16(_ptr(b), _ptr(sc), _ptr(out), ctypes.c_int64(sc.numel()))
        return out.to(out_dtype)
    lut = _E2M1_VALUES.to(blocks.device)
    lo, hi = (blocks & 0x0F).long(), (blocks >> 4).long()
    vals = torch.stack([lut[lo], lut[hi]], dim=-1).flatten(-2)            # [..., G, 32]
    exp = torch.exp2(scales.float() - 127.0).unsqueeze(-1)
    return (vals * exp).flatten(-2).to(out_dtype)


def quant_mxfp4(x: torch.Tensor, native: bool = True):
    """Inverse of ``dequant_mxfp4`` (round to nearest e2m1 under a power-of-two group scale); x: [..., 32*G]."""
    if native and _on_host(x):
        import ctypes

        xf = x.float().contiguous()
        G = xf.shape[-1] // 32
        blocks = torch.empty(tuple(xf.shape[:-1]) + (G, 16), dtype=torch.uint8)
        scales = torch.empty(tuple(xf.shape[:-1]) + (G,), dtype=torch.uint8)
        _host_lib().pfb_mxfp4_quant(_ptr(xf), _ptr(blocks), _ptr(scales), ctypes.c_int64(scales.numel()))
        return blocks, scales
    g = x.float().unflatten(-1, (-1, 32))
    amax = g.abs().amax(-1, keepdim=True).clamp(min=2.0 ** -126)
    m, k = torch.frexp(amax / 6.0)                        # exact ceil(log2(.)): no rounding of a logarithm
    e = torch.where(m > 0.5, k, k - 1).float()
    scaled = g / torch.exp2(e)
    lut = _E2M1_VALUES.to(x.device)
    idx = (scaled.unsqueeze(-1) - lut).abs().argmin(-1)
    blocks = (idx[..., 0::2] | (idx[..., 1::2] << 4)).to(torch.uint8)
    return blocks, (e.squeeze(-1) + 127).clamp(0, 255).to(torch.uint8)


def dequant_mxfp8(q: torch.Tensor, scales: torch.Tensor, out_dtype=torch.bfloat16, native: bool = True) -> torch.Tensor:
    """q: e4m3 (or its uint8 view) [..., 32*G]; scales: uint8 [..., G] E8M0, one per group of 32 values."""
    if native and _on_host(q, scales):
        import ctypes

        qq, sc = q.contiguous().view(torch.uint8), scales.contiguous()
        out = torch.empty(qq.shape, dtype=torch.bfloat16)
        _host_lib().pfb_mxfp8_dequant_bf16(_ptr(qq), _ptr(sc), _ptr(out), ctypes.c_int64(sc.numel()))
        return out.to(out_dtype)
    vals = (q if q.dtype == torch.float8_e4m3fn else q.view(torch.float8_e4m3fn)).float().unflatten(-1, (-1, 32))
    return (vals * torch.exp2(scales.float() - 127.0).unsqueeze(-1)).flatten(-2).to(out_dtype)


def quant_mxfp8(x: torch.Tensor, native: bool = True):
    """x [..., 32*G] -> (e4m3 [..., 32*G], E8M0 uint8 [..., G]): the group's power-of-two scale maps its largest magnitude
    into the e4m3 range (<= 448), values round to nearest even."""
    if native and _on_host(x):
        import ctypes

        xf = x.float().contiguous()
        q = torch.empty(xf.shape, dtype=torch.uint8)
        scales = torch.empty(tuple(xf.shape[:-1]) + (xf.shape[-1] // 32,), dtype=torch.uint8)
        _host_lib().pfb_mxfp8_quant(_ptr(xf), _ptr(q), _ptr(scales), ctypes.c_int64(scales.numel()))
        return q.view(torch.float8_e4m3fn), scales
    g = x.float().unflatten(-1, (-1, 32))
    amax = g.abs().amax(-1, keepdim=True).clamp(min=2.0 ** -126)
    m, k = torch.frexp(amax / 448.0)                      # exact ceil(log2(.)): no rounding of a logarithm
    e = torch.where(m > 0.5, k, k - 1).clamp(-127, 127)
    q = (g * torch.exp2(-e.float())).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).flatten(-2)
    return q, (e.squeeze(-1) + 127).to(torch.uint8)


def downcast_to_mxfp(x: torch.Tensor, fmt: str = "mxfp4"):
    """(values, scales) of ``x`` in a micro-scaled format: groups of 32 along the last dimension, one E8M0 scale each
    (paddleformers/utils/upcast_downcast_triton.py: ``_downcast_to_mxfp``)."""
    if fmt == "mxfp4":
        return quant_mxfp4(x)
    if fmt == "mxfp8":
        return quant_mxfp8(x)
    raise ValueError(f"unknown micro-scaled format {fmt!r} (mxfp4, mxfp8)")


def upcast_from_mxfp(values: torch.Tensor, scales: torch.Tensor, fmt: str = "mxfp4", dtype=torch.bfloat16) -> torch.Tensor:
    """Inverse of ``downcast_to_mxfp`` (``_upcast_from_mxfp`` in the reference)."""
    if fmt == "mxfp4":
        return dequant_mxfp4(values, scales, dtype)
    if fmt == "mxfp8":
        return dequant_mxfp8(values, scales, dtype)
    raise ValueError(f"unknown micro-scaled format {fmt!r} (mxfp4, mxfp8)")


class MXFP4Reader:
    """Checkpoint reader view for MXFP4 checkpoints (gpt-oss): a tensor stored as ``<name>_blocks`` (uint8
    [..., rows, groups, 16]) with ``<name>_scales`` ([..., rows, groups]) appears under ``<name>`` as the de-quantised bf16
    tensor. The quantised axis is the input dimension of each projection and is stored last, while the unquantised format
    of these tensors is [experts, in, out]: the de-quantised tensor is therefore transposed to that layout
    (paddleformers/quantization/checkpoint_dequant.py:295-355)."""

    def __init__(self, reader):
        self.reader = reader

    def __getattr__(self, name):
        return getattr(self.reader, name)

    def has(self, name: str) -> bool:
        return self.reader.has(name) or (self.reader.has(name + "_blocks") and self.reader.has(name + "_scales"))

    def get(self, name: str) -> torch.Tensor:
        if self.reader.has(name):
            return self.reader.get(name)
        full = dequant_mxfp4(self.reader.get(name + "_blocks"), self.reader.get(name + "_scales"))   # [..., rows, in]
        return full.transpose(-1, -2).contiguous() if full.dim() >= 3 else full


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
