"""Quantisation, checkpoint de-quantisation and model merging."""
import os

import torch

from paddleformers_b200.quantization.checkpoint_dequant import dequant_fp8_block, dequant_mxfp4, quant_mxfp4
from paddleformers_b200.quantization.fp8 import (FP8Linear, dequant_act, dequant_weight, fp8_gemm_reference, quant_act_1x128,
                                                 quant_weight_128x128)
from paddleformers_b200.quantization.weight_only import QuantizationLinear


def test_fp8_block_quant_roundtrip_and_gemm():
    torch.manual_seed(0)
    x, w = torch.randn(37, 300), torch.randn(200, 300)
    for ue8m0 in (False, True):
        xq, xs = quant_act_1x128(x, ue8m0)
        wq, ws = quant_weight_128x128(w, ue8m0)
        assert xs.shape == (37, 3) and ws.shape == (2, 3)
        if ue8m0:
            assert torch.equal(torch.log2(xs), torch.log2(xs).round())
        assert ((dequant_act(xq, xs) - x).norm() / x.norm()) < 0.05
        assert ((dequant_weight(wq, ws) - w).norm() / w.norm()) < 0.05
        y = fp8_gemm_reference(xq, xs, wq, ws)
        assert ((y - x @ w.t()).norm() / (x @ w.t()).norm()) < 0.06
    assert torch.allclose(dequant_fp8_block(wq, ws).float(), dequant_weight(wq, ws), atol=0.05, rtol=0.02)


def test_fp8_linear_trains():
    torch.manual_seed(1)
    lin = FP8Linear(256, 128, dtype=torch.float32)
    x = torch.randn(16, 256, requires_grad=True)
    y = lin(x)
    y.sum().backward()
    ref = torch.nn.functional.linear(x, lin.weight)
    assert ((y - ref).norm() / ref.norm()) < 0.06 and lin.weight.grad is not None and x.grad is not None


def test_mxfp4_roundtrip():
    torch.manual_seed(2)
    x = torch.randn(4, 64)
    blocks, scales = quant_mxfp4(x)
    assert blocks.shape == (4, 2, 16) and scales.shape == (4, 2)
    back = dequant_mxfp4(blocks, scales, torch.float32)
    assert ((back - x).norm() / x.norm()) < 0.25
    b2, s2 = quant_mxfp4(back)
    assert torch.equal(dequant_mxfp4(b2, s2, torch.float32), back)   # representable values are fixed points


def test_weight_only_linears():
    torch.manual_seed(3)
    lin = torch.nn.Linear(128, 64)
    x = torch.randn(5, 128)
    for algo, tol in (("wint8", 0.02), ("wint4", 0.2), ("nf4", 0.15)):
        q = QuantizationLinear(lin, algo)
        assert ((q(x) - lin(x)).norm() / lin(x).norm()) < tol


def test_merge_methods(tmp_path):
    from safetensors.torch import load_file, save_file

    from paddleformers_b200.mergekit import MergeConfig, MergeModel

    torch.manual_seed(4)
    base = {"a.weight": torch.randn(8, 8), "b.weight": torch.randn(4)}
    m1 = {k: v + 0.1 * torch.randn_like(v) for k, v in base.items()}
    m2 = {k: v + 0.1 * torch.randn_like(v) for k, v in base.items()}
    for name, sd in (("base", base), ("m1", m1), ("m2", m2)):
        os.makedirs(tmp_path / name)
        save_file(sd, str(tmp_path / name / "model.safetensors"))
        (tmp_path / name / "config.json").write_text("{}")
    paths = [str(tmp_path / "m1"), str(tmp_path / "m2")]
    out = MergeModel(MergeConfig("linear", paths, weight_list=[1, 3], output_path=str(tmp_path / "lin"))).merge()
    got = load_file(os.path.join(out, "model.safetensors"))
    assert torch.allclose(got["a.weight"], 0.25 * m1["a.weight"] + 0.75 * m2["a.weight"], atol=1e-6)
    out = MergeModel(MergeConfig("slerp", paths, slerp_t=0.0, output_path=str(tmp_path / "sl"))).merge()
    assert torch.allclose(load_file(os.path.join(out, "model.safetensors"))["a.weight"], m1["a.weight"], atol=1e-5)
    out = MergeModel(MergeConfig("ties", paths, base_model_path=str(tmp_path / "base"), reserve_p=1.0, sparsify_type="trim",
                                 output_path=str(tmp_path / "ties"))).merge()
    t = load_file(os.path.join(out, "model.safetensors"))["a.weight"]
    d1, d2 = m1["a.weight"] - base["a.weight"], m2["a.weight"] - base["a.weight"]
    same = torch.sign(d1) == torch.sign(d2)
    assert torch.allclose(t[same], (base["a.weight"] + (d1 + d2) / 2)[same], atol=1e-5)
    assert os.path.exists(os.path.join(out, "config.json"))


def test_qat_linears_hadamard_and_qlora():
    import torch.nn as nn

    from paddleformers_b200.peft.lora import LoRAConfig, LoRAModel
    from paddleformers_b200.quantization.qat import (QATLinear, block_hadamard, convert_to_qat, fake_quant_per_token,
                                                     hadamard_transform)
    from paddleformers_b200.quantization.weight_only import quantize_model

    torch.manual_seed(0)
    x = torch.randn(7, 64)
    # Hadamard: orthonormal and an involution
    h = hadamard_transform(x)
    assert torch.allclose(hadamard_transform(h), x, atol=1e-5) and torch.allclose(h.norm(dim=-1), x.norm(dim=-1), atol=1e-4)
    assert torch.allclose(block_hadamard(block_hadamard(x, 16), 16), x, atol=1e-5)
    # fake quantisation: at most half a step of error, gradients pass through
    xq = fake_quant_per_token(x.clone().requires_grad_(True))
    step = x.abs().amax(-1, keepdim=True) / 127
    assert ((xq - x).abs() <= step / 2 + 1e-6).all()
    lin = nn.Linear(64, 32)
    q = QATLinear(lin, hadamard_block=16)
    xin = x.clone().requires_grad_(True)
    y = q(xin)
    assert (y - lin(x)).abs().max() < 0.05
    y.sum().backward()
    assert lin.weight.grad is not None and xin.grad.abs().sum() > 0
    # QLoRA: adapters on top of nf4 bases; only the adapters train
    net = nn.Sequential()
    net.add_module("qkv_proj", nn.Linear(64, 64))
    net.add_module("down_proj", nn.Linear(64, 64))
    assert quantize_model(net, "nf4") == 2
    lora = LoRAModel(net, LoRAConfig(r=4, lora_alpha=8))
    names = [n for n, p in lora.named_parameters() if p.requires_grad]
    assert len(names) == 4 and all("lora_" in n for n in names)
    out = lora(x)
    out.sum().backward()
    assert all(p.grad is not None for n, p in lora.named_parameters() if p.requires_grad)
    m2 = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 8))
    assert convert_to_qat(m2, "a8w4") == 2


def test_native_block_scaled_converters_match_the_tensor_implementations():
    """The compiled host converters against the tensor-op specification: bit-identical codes, scales and values."""
    from paddleformers_b200.ops._build import build_host_library
    from paddleformers_b200.quantization import checkpoint_dequant as cd

    build_host_library()
    cd._host = None
    assert cd._host_lib() is not None
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 256, generator=g) * torch.logspace(-6, 4, 64).unsqueeze(1)      # many magnitudes
    x[3, :32] = 0.0
    x[5, 7] = 6.0 * 2.0 ** 3                                                             # exactly on a scale boundary
    # mxfp4
    bn, sn = cd.quant_mxfp4(x, native=True)
    bt, st = cd.quant_mxfp4(x, native=False)
    assert torch.equal(sn, st) and torch.equal(bn, bt)
    assert torch.equal(cd.dequant_mxfp4(bn, sn, torch.float32, native=True), cd.dequant_mxfp4(bn, sn, torch.float32, native=False))
    # mxfp8
    qn, s8n = cd.quant_mxfp8(x, native=True)
    qt, s8t = cd.quant_mxfp8(x, native=False)
    assert torch.equal(s8n, s8t) and torch.equal(qn.view(torch.uint8), qt.view(torch.uint8))
    back = cd.dequant_mxfp8(qn, s8n, torch.float32, native=True)
    assert torch.equal(back, cd.dequant_mxfp8(qn, s8n, torch.float32, native=False))
    nz = x.abs() > 1e-3 * x.abs().amax(-1, keepdim=True)
    assert ((back - x).abs()[nz] / x.abs()[nz]).max() < 0.07                              # e4m3: 3 mantissa bits
    # every e4m3 byte decodes like torch's own conversion
    allb = torch.arange(256, dtype=torch.uint8).repeat(1, 1)
    sc = torch.full((1, 8), 127, dtype=torch.uint8)
    mine = cd.dequant_mxfp8(allb, sc, torch.float32, native=True)
    ref = allb.view(torch.float8_e4m3fn).float()
    ok = ~ref.isnan()
    assert torch.equal(mine[ok], ref[ok]) and mine[~ok].isnan().all()
    # names of the reference's converters
    v, s = cd.downcast_to_mxfp(x, "mxfp4")
    assert torch.equal(cd.upcast_from_mxfp(v, s, "mxfp4", torch.float32), cd.dequant_mxfp4(bn, sn, torch.float32))
    # fp8 128x128 block checkpoints
    w = (torch.randn(200, 300, generator=g)).to(torch.float8_e4m3fn)
    scale = torch.rand(2, 3, generator=g) + 0.5
    assert torch.equal(cd.dequant_fp8_block(w, scale, 128, native=True), cd.dequant_fp8_block(w, scale, 128, native=False))
