"""Block-scaled fp8 kernels (quantisation, tcgen05 e4m3 GEMM, grouped variant, FP8Linear) against fp32 PyTorch math."""
import pytest
import torch

from paddleformers_b200.quantization import fp8 as Q

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("ue8m0", [True, False])
def test_quant_kernels_match_reference(ue8m0):
    torch.manual_seed(0)
    x = (torch.randn(300, 512, device="cuda") * torch.rand(300, 1, device="cuda") * 4).to(torch.bfloat16)
    x[5] = 0                                                       # an all-zero block
    q, s_t = Q.quant_act_kernel(x, ue8m0)
    q_ref, s_ref = Q.quant_act_1x128(x, ue8m0)
    assert q.shape == (300, 512) and s_t.shape == (4, 300)
    torch.testing.assert_close(s_t.t(), s_ref, rtol=1e-6, atol=0)
    assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean().item() < 1e-3   # division rounding at ties only
    torch.testing.assert_close(Q.dequant_act(q, s_t.t()), Q.dequant_act(q_ref, s_ref), rtol=0.13, atol=1e-6)   # where they differ it is by one e4m3 step

    w = (torch.randn(200, 384, device="cuda") * 0.05).to(torch.bfloat16)     # 200 rows: a ragged last block
    wq, ws = Q.quant_weight_kernel(w, ue8m0)
    wq_ref, ws_ref = Q.quant_weight_128x128(w, ue8m0)
    assert ws.shape == (2, 3)
    torch.testing.assert_close(ws, ws_ref, rtol=1e-6, atol=0)
    assert (wq.view(torch.uint8) != wq_ref.view(torch.uint8)).float().mean().item() < 1e-3


# pow2 = True: power-of-two scales applied by the tensor core (tiles 128 / 192 / 240 wide, chosen from N);
# pow2 = False: arbitrary fp32 scales promoted in the epilogue
@pytest.mark.parametrize("pow2", [True, False])
@pytest.mark.parametrize("M,N,K", [(300, 384, 512), (128, 128, 128), (1024, 1536, 7168), (77, 200, 256), (512, 4096, 640),
                                   (2048, 720, 1024)])
def test_fp8_gemm_matches_reference(M, N, K, pow2):
    torch.manual_seed(1)
    x = (torch.randn(M, K, device="cuda") * torch.rand(M, 1, device="cuda") * 8).to(torch.bfloat16)   # scales differ by row
    w = (torch.randn(N, K, device="cuda") * torch.rand(N, 1, device="cuda") * 0.1).to(torch.bfloat16)
    xq, xs_t = Q.quant_act_kernel(x, pow2)
    wq, ws = Q.quant_weight_kernel(w, pow2)
    out = Q.fp8_gemm(xq, xs_t, wq, ws, pow2=pow2)
    ref = Q.fp8_gemm_reference(xq, xs_t.t(), wq, ws)
    assert _rel(out, ref) < 6e-3                                   # bf16 rounding of the output
    assert _rel(out, x.float() @ w.float().t()) < 6e-2             # and the quantisation error itself stays small
    from paddleformers_b200.ops import functional as F

    F.check_kernel_status()


@pytest.mark.parametrize("N", [256, 384, 1200])
def test_fp8_grouped_gemm(N):
    torch.manual_seed(2)
    E, K = 4, 512
    block_expert = torch.tensor([2, 0, -1, 3, 3, 1], dtype=torch.int32, device="cuda")
    M = block_expert.numel() * 128
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(E * N, K, device="cuda") * torch.rand(E * N, 1, device="cuda") * 0.1).to(torch.bfloat16)
    xq, xs_t = Q.quant_act_kernel(x)
    wq, ws = Q.quant_weight_kernel(w)
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    Q.fp8_gemm(xq, xs_t, wq, ws, block_expert=block_expert, n_per_expert=N, out=out)
    xd = Q.dequant_act(xq, xs_t.t())
    wd = Q.dequant_weight(wq, ws)
    for b, e in enumerate(block_expert.tolist()):
        rows = slice(b * 128, (b + 1) * 128)
        if e < 0:
            assert out[rows].abs().max().item() == 0
        else:
            assert _rel(out[rows], xd[rows] @ wd[e * N:(e + 1) * N].t()) < 6e-3


def test_scales_that_are_not_powers_of_two_are_refused_by_the_tensor_core_path():
    from paddleformers_b200.ops import functional as F

    s = torch.full((2, 256), 0.75, device="cuda")
    torch.ops.pfb200.mx_pack_scales(s, True, 256, 1, 128)
    with pytest.raises(RuntimeError):
        F.check_kernel_status()
    F.check_kernel_status()          # the status word was reset by the failed check


@pytest.mark.parametrize("weighted", [False, True])
def test_fused_swiglu_quant_forward_and_backward(weighted):
    """act = prob * silu(gate) * up quantised in one pass, and its backward with quantised gate / up gradients, against
    fp32 autograd followed by the reference quantiser."""
    torch.manual_seed(6)
    R, I = 300, 384
    gu = torch.randn(R, 2 * I, device="cuda", dtype=torch.bfloat16)
    prob = torch.rand(R, device="cuda") if weighted else None
    dact = torch.randn(R, I, device="cuda", dtype=torch.bfloat16)
    q, s_t, act = torch.ops.pfb200.swiglu_quant_fwd(gu, prob, True, True)
    guf = gu.float().requires_grad_()
    pf = prob.clone().requires_grad_() if weighted else None
    ref = torch.nn.functional.silu(guf[:, :I]) * guf[:, I:] * (pf[:, None] if weighted else 1.0)
    ref.backward(dact.float())
    assert _rel(act, ref) < 5e-3
    assert _rel(Q.dequant_act(q, s_t.t()), ref) < 4e-2            # e4m3 has three mantissa bits
    q_ref, s_ref = Q.quant_act_1x128(ref.detach(), True)
    torch.testing.assert_close(s_t.t(), s_ref, rtol=1e-6, atol=0)
    dgu, gq, gs_t, act2, dpp = torch.ops.pfb200.swiglu_quant_bwd(dact, gu, prob, True, True)
    assert _rel(dgu, guf.grad) < 5e-3 and _rel(act2, ref) < 5e-3
    assert _rel(Q.dequant_act(gq, gs_t.t()), guf.grad) < 4e-2
    if weighted:
        assert _rel(dpp.sum(0), pf.grad) < 1e-3
    else:
        assert dpp.numel() == 0


def test_transposing_quantiser_and_fp8_weight_gradient():
    torch.manual_seed(7)
    T, N, K = 1000, 384, 512                                      # T is not a multiple of 128: the tail is zero-filled
    x = (torch.randn(T, K, device="cuda") * torch.rand(1, K, device="cuda") * 4).to(torch.bfloat16)
    dy = (torch.randn(T, N, device="cuda") * 0.02).to(torch.bfloat16)
    q_t, s = Q.quant_transpose_kernel(x)
    assert q_t.shape == (K, 1024) and s.shape == (8, K)
    xp = torch.nn.functional.pad(x.float(), (0, 0, 0, 24))
    q_ref, s_ref = Q.quant_act_1x128(xp.t().contiguous(), True)   # [K, 1024] with 1x128 blocks along tokens
    torch.testing.assert_close(s.t(), s_ref, rtol=1e-6, atol=0)
    assert (q_t.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean().item() < 1e-3
    ref = dy.float().t() @ x.float()
    dw = Q.fp8_wgrad(dy, x)
    assert _rel(dw, ref) < 6e-2
    acc = torch.ones(N, K, device="cuda")
    Q.fp8_wgrad(dy, x, acc)
    torch.testing.assert_close(acc, dw + 1.0, rtol=1e-5, atol=1e-5)
    from paddleformers_b200.ops import functional as F

    F.check_kernel_status()


def test_fp8_linear_forward_backward():
    torch.manual_seed(3)
    lin = Q.FP8Linear(512, 384, dtype=torch.bfloat16, device="cuda")
    x = torch.randn(4, 64, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = lin(x)
    g = torch.randn_like(y)
    y.backward(g)
    w = lin.weight.detach().float()
    assert _rel(y, x.detach().float() @ w.t()) < 6e-2
    assert _rel(x.grad, g.float() @ w) < 6e-2
    assert _rel(lin.weight.grad, g.float().reshape(-1, 384).t() @ x.detach().float().reshape(-1, 512)) < 6e-2   # fp8 wgrad


def test_fp8_grouped_experts_match_bf16_experts():
    """Expert MLP on block-scaled fp8 GEMMs (forward and input gradients) against the bf16 grouped kernels."""
    from paddleformers_b200.models.configuration import Qwen3MoeConfig
    from paddleformers_b200.nn.moe import GroupedExperts

    torch.manual_seed(4)
    kw = dict(hidden_size=256, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128, intermediate_size=128,
              num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, vocab_size=64)
    ref = GroupedExperts(Qwen3MoeConfig(**kw), dtype=torch.bfloat16, device="cuda")
    cfg8 = Qwen3MoeConfig(**kw)
    cfg8.fp8 = "e4m3"
    low = GroupedExperts(cfg8, dtype=torch.bfloat16, device="cuda")
    assert low.use_fp8 and not ref.use_fp8
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, 0.05)
        low.gate_up_proj.copy_(ref.gate_up_proj)
        low.down_proj.copy_(ref.down_proj)
    # the dispatcher's layout: expert segments in ascending order, unowned blocks (-1) behind them
    block_expert = torch.tensor([0, 1, 1, 2, 3, -1], dtype=torch.int32, device="cuda")
    R = block_expert.numel() * 128
    x = torch.randn(R, 256, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(R, 256, device="cuda", dtype=torch.bfloat16)
    g[5 * 128:] = 0                                            # rows of the unowned block carry no gradient
    outs = []
    for mod in (ref, low):
        xi = x.clone().requires_grad_(True)
        y = mod(xi, block_expert)
        y.backward(g)
        outs.append((y.detach(), xi.grad.detach(), mod.gate_up_proj.grad.detach().clone(), mod.down_proj.grad.detach().clone()))
    live = torch.cat([torch.arange(b * 128, (b + 1) * 128) for b, e in enumerate(block_expert.tolist()) if e >= 0]).cuda()
    for name, a, b in zip(("y", "dx"), outs[1][:2], outs[0][:2]):
        assert _rel(a[live], b[live]) < 8e-2, name
    for name, a, b in zip(("dw_gate_up", "dw_down"), outs[1][2:], outs[0][2:]):
        assert _rel(a, b) < 8e-2, name
    from paddleformers_b200.ops import functional as F

    F.check_kernel_status()
