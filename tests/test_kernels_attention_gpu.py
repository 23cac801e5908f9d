"""tcgen05 flash attention against an fp32 PyTorch reference (causal, GQA, document masks)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(scope="module")
def F():
    from paddleformers_b200.ops import functional as F

    return F


def _doc_kend(B, S, device, seed):
    g = torch.Generator().manual_seed(seed)
    kend = torch.empty(B, S, dtype=torch.int32)
    for b in range(B):
        pos = 0
        while pos < S:
            ln = int(torch.randint(16, 300, (1,), generator=g))
            end = min(S, pos + ln)
            kend[b, pos:end] = end
            pos = end
    return kend.to(device)


@pytest.mark.parametrize("p_in_tmem", [True, False])
@pytest.mark.parametrize("B,S,Hq,Hkv,docs", [(1, 128, 2, 2, False), (2, 512, 4, 2, False), (1, 640, 4, 1, True), (1, 200, 2, 1, False)])
def test_attention_forward(F, p_in_tmem, B, S, Hq, Hkv, docs):
    torch.manual_seed(0)
    F.set_attention_options(p_in_tmem=p_in_tmem)
    q = torch.randn(B, S, Hq, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16)
    kend = _doc_kend(B, S, "cuda", 1) if docs else None
    out = F.flash_attention(q, k, v, causal=True, kend=kend)
    F.check_kernel_status()
    ref = F.attention_reference(q, k, v, causal=True, kend=kend)
    F.set_attention_options(p_in_tmem=True)
    assert _rel_err(out, ref) < 2e-2


def _backward_case(F, B, S, Hq, Hkv, causal, docs, seed=1):
    torch.manual_seed(seed)
    q = torch.randn(B, S, Hq, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    kend = _doc_kend(B, S, "cuda", 2) if docs else None
    out = F.flash_attention(q, k, v, causal=causal, kend=kend)
    g = torch.randn_like(out)
    out.backward(g)
    F.check_kernel_status()
    return q, k, v, kend, out, g


# heads_per_cta: 1 = one CTA per query head (fp32 dK / dV partials), 2 = one CTA per KV head walking its query heads
@pytest.mark.parametrize("hpc", [1, 2])
@pytest.mark.parametrize("B,S,Hq,Hkv,causal,docs", [
    (1, 384, 4, 2, True, True),      # documents, G = 2
    (2, 512, 4, 4, True, False),     # batch 2, G = 1
    (1, 456, 4, 1, True, False),     # S not a multiple of 64, G = 4
    (1, 320, 8, 1, False, False),    # not causal, G = 8
    (2, 200, 2, 1, False, True),     # not causal + documents, ragged, batch 2
    (1, 1024, 8, 2, True, True),     # many tiles per CTA: exercises every ring wrap
])
def test_attention_backward(F, hpc, B, S, Hq, Hkv, causal, docs):
    F.set_attention_options(bwd_heads_per_cta=hpc)
    try:
        q, k, v, kend, out, g = _backward_case(F, B, S, Hq, Hkv, causal, docs)
    finally:
        F.set_attention_options(bwd_heads_per_cta=0)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = F.attention_reference(qr, kr, vr, causal=causal, kend=kend)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 2e-2
    assert _rel_err(q.grad, qr.grad) < 3e-2 and _rel_err(k.grad, kr.grad) < 3e-2 and _rel_err(v.grad, vr.grad) < 3e-2


def test_attention_backward_deterministic_mode_is_bitwise_reproducible(F):
    """With ordered dQ accumulation two runs on the same inputs give identical bits (the default adds the key tiles'
    contributions in arrival order)."""
    F.set_attention_options(deterministic=True)
    try:
        runs = []
        for _ in range(2):
            q, k, v, kend, out, g = _backward_case(F, 2, 1024, 8, 2, True, True, seed=5)
            runs.append((q.grad.clone(), k.grad.clone(), v.grad.clone()))
        qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
        ref = F.attention_reference(qr, kr, vr, causal=True, kend=kend)
        ref.backward(g.float())
    finally:
        F.set_attention_options(deterministic=False)
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    assert _rel_err(runs[0][0], qr.grad) < 3e-2 and _rel_err(runs[0][1], kr.grad) < 3e-2


@pytest.mark.parametrize("B,S,H,causal,docs", [(1, 384, 4, True, False), (2, 200, 2, True, True), (1, 520, 3, False, False)])
def test_latent_attention_192_wide_keys_128_wide_values(F, B, S, H, causal, docs):
    """Multi-head latent attention shapes (queries / keys 192 wide, values 128 wide) on the tcgen05 kernels, forward and
    backward, against the fp32 reference."""
    torch.manual_seed(4)
    q = torch.randn(B, S, H, 192, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, S, H, 192, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, S, H, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    kend = _doc_kend(B, S, "cuda", 3) if docs else None
    out = F.flash_attention(q, k, v, causal=causal, kend=kend)
    assert out.shape == (B, S, H, 128)
    g = torch.randn_like(out)
    out.backward(g)
    F.check_kernel_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = F.attention_reference(qr, kr, vr, causal=causal, kend=kend)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 2e-2
    assert _rel_err(q.grad, qr.grad) < 3e-2 and _rel_err(k.grad, kr.grad) < 3e-2 and _rel_err(v.grad, vr.grad) < 3e-2
