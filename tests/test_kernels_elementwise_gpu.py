"""Memory-bound kernels against fp32 PyTorch references."""
import math

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


@pytest.mark.parametrize("T,H", [(64, 256), (333, 4096), (17, 7168)])
def test_rms_norm_fwd_bwd(F, T, H):
    torch.manual_seed(0)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = F.rms_norm(x, w, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


def test_rms_norm_residual(F):
    torch.manual_seed(1)
    T, H = 100, 512
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y, s = F.rms_norm(x, w, 1e-6, residual=r)
    gy, gs = torch.randn_like(y), torch.randn_like(s)
    (y * gy).sum().add((s * gs).sum()).backward()
    xr, rr = x.detach().float().requires_grad_(), r.detach().float().requires_grad_()
    sr = (xr + rr).to(torch.bfloat16).float() + 0 * (xr + rr)  # same rounding of the sum
    sr = xr + rr
    yr = sr * torch.rsqrt(sr.pow(2).mean(-1, keepdim=True) + 1e-6)
    ((yr * gy.float()).sum() + (sr * gs.float()).sum()).backward()
    assert _rel_err(s, sr) < 1e-2 and _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 2e-2 and _rel_err(r.grad, rr.grad) < 2e-2


def test_swiglu(F):
    torch.manual_seed(2)
    gu = torch.randn(77, 2 * 328, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = F.swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    gr = gu.detach().float().requires_grad_()
    a, b = gr.chunk(2, -1)
    yr = torch.nn.functional.silu(a) * b
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(gu.grad, gr.grad) < 1e-2


@pytest.mark.parametrize("rot", [128, 64])
def test_rope_and_qk_norm(F, rot):
    torch.manual_seed(3)
    T, nh, D = 50, 6, 128
    cos, sin = F.rope_tables(256, rot, 10000.0, "cuda")
    pos = torch.randint(0, 256, (T,), device="cuda")
    x = torch.randn(T, nh * D + 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = F.rope_heads(x, cos, sin, pos, nh, D, rot)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = F._rope_ref(xr[:, : nh * D].reshape(T, nh, D), cos, sin, pos, rot).reshape(T, nh * D)
    yr = torch.cat([yr, xr[:, nh * D:]], -1)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2
    # qk-norm + rope
    nw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_()
    x2 = torch.randn(T, nh * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y2 = F.qk_norm_rope(x2, nw, cos, sin, pos, nh, D, rot, 1e-6)
    g2 = torch.randn_like(y2)
    y2.backward(g2)
    x2r = x2.detach().float().requires_grad_()
    nwr = nw.detach().float().requires_grad_()
    h = x2r.reshape(T, nh, D)
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6) * nwr
    y2r = F._rope_ref(h, cos, sin, pos, rot).reshape(T, nh * D)
    y2r.backward(g2.float())
    assert _rel_err(y2, y2r) < 1e-2 and _rel_err(x2.grad, x2r.grad) < 2e-2 and _rel_err(nw.grad, nwr.grad) < 2e-2


def test_embedding(F):
    torch.manual_seed(4)
    V, H = 1000, 256
    w = torch.randn(V, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, V, (3, 70), device="cuda")
    out = F.embedding(ids, w)
    assert torch.equal(out, w.detach()[ids])
    g = torch.randn_like(out)
    out.backward(g)
    ref = torch.zeros(V, H, device="cuda").index_add_(0, ids.reshape(-1), g.reshape(-1, H).float())
    assert _rel_err(w.grad, ref) < 1e-2
    # vocabulary shard
    shard = F.embedding(ids, w.detach()[200:600].contiguous(), vocab_start=200)
    mask = ((ids >= 200) & (ids < 600))[..., None]
    assert torch.equal(shard, w.detach()[ids] * mask)


@pytest.mark.parametrize("V", [1024, 32000])
def test_fused_linear_cross_entropy(F, V):
    torch.manual_seed(5)
    T, H = 300, 256
    h = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, H, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    scale = torch.tensor(1.0 / 200, device="cuda")
    loss, cnt = F.fused_linear_cross_entropy(h, w, labels, chunk=128, loss_scale=scale)
    loss.backward()
    hr = h.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    lr = torch.nn.functional.cross_entropy(hr @ wr.t(), labels, ignore_index=-100, reduction="sum") / 200
    lr.backward()
    assert int(cnt) == int((labels != -100).sum())
    assert abs(loss.item() - lr.item()) / abs(lr.item()) < 5e-3
    assert _rel_err(h.grad, hr.grad) < 3e-2 and _rel_err(w.grad, wr.grad) < 3e-2


def test_adamw_and_sq_norm(F):
    torch.manual_seed(6)
    n = 100003
    ops = torch.ops.pfb200
    p = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    g = torch.randn(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ref_p = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        ref_p.grad = g.clone() * 0.5
        opt.step()
        scalars = torch.tensor([1e-2, 0.5, 1 - 0.9 ** step, 1 - 0.95 ** step, 0.0], device="cuda")
        ops.adamw_step(p, m, v, g, p16, scalars, 0.9, 0.95, 1e-8, 0.1)
    assert _rel_err(p, ref_p.detach()) < 1e-5
    assert _rel_err(p16, ref_p.detach()) < 1e-2
    out = torch.zeros(1, device="cuda")
    scratch = torch.empty(int(ops.sq_norm_scratch_elems()), device="cuda")
    ops.sq_norm_accum(g, out, scratch)
    assert abs(out.item() - g.double().pow(2).sum().item()) / g.double().pow(2).sum().item() < 1e-5
