"""tcgen05 GEMM numerics against fp32 PyTorch references (all operand layouts and epilogues)."""
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


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (384, 1024, 4096), (200, 328, 136), (4096, 1024, 1024),
                                   (1000, 1304, 520), (4096, 6144, 4096)])
@pytest.mark.parametrize("bn", [128, 256, 0])   # 0 = automatic: the CTA-pair kernel when the shape has 256 x 256 tiles
def test_gemm_nt(F, M, N, K, bn):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = F.gemm(a, b, force_bn=bn)
    F.check_kernel_status()
    ref = a.float() @ b.float().t()
    assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("bn", [128, 256, 0])   # 0 = automatic: the CTA-pair kernel when the shape has 256 x 256 tiles
def test_gemm_dgrad_layout(F, bn):
    torch.manual_seed(1)
    M, N, K = 512, 384, 640  # dx[M,N] = dy[M,K] @ W[K,N]
    dy = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    out = F.gemm(dy, w, b_mn=True, force_bn=bn)
    F.check_kernel_status()
    assert _rel_err(out, dy.float() @ w.float()) < 1e-2


@pytest.mark.parametrize("bn", [128, 256, 0])   # 0 = automatic: the CTA-pair kernel when the shape has 256 x 256 tiles
def test_gemm_wgrad_layout_accumulate(F, bn):
    torch.manual_seed(2)
    T, O, I = 1024, 384, 512  # dW[O,I] = dy[T,O]^T @ x[T,I]
    dy = torch.randn(T, O, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    acc = torch.randn(O, I, device="cuda", dtype=torch.float32)
    ref = acc + dy.float().t() @ x.float()
    F.gemm(dy, x, out=acc, a_mn=True, b_mn=True, epi=F.EPI_ACCUM_F32, force_bn=bn)
    F.check_kernel_status()
    assert _rel_err(acc, ref) < 1e-3
    out = F.gemm(dy, x, a_mn=True, b_mn=True, epi=F.EPI_STORE_BF16, force_bn=bn)
    assert _rel_err(out, dy.float().t() @ x.float()) < 1e-2


@pytest.mark.parametrize("bn", [128, 256, 0])   # 0 = automatic: the CTA-pair kernel when the shape has 256 x 256 tiles
def test_gemm_swiglu_epilogue(F, bn):
    torch.manual_seed(3)
    T, H, I = 512, 256, 384
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(2 * I, H, device="cuda", dtype=torch.bfloat16) * 0.1
    raw = torch.empty(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    act = F.gemm(x, w, epi=F.EPI_SWIGLU_BF16, out2=raw, force_bn=bn)
    F.check_kernel_status()
    gu = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    assert _rel_err(raw, gu) < 1e-2
    assert _rel_err(act, ref) < 2e-2


def test_gemm_residual_accumulate(F):
    torch.manual_seed(4)
    a = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(384, 512, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16)
    ref = res.float() + a.float() @ b.float().t()
    F.gemm(a, b, out=res, epi=F.EPI_ACCUM_BF16)
    F.check_kernel_status()
    assert _rel_err(res, ref) < 1e-2


@pytest.mark.parametrize("bn", [128, 256, 0])   # 0 = automatic: the CTA-pair kernel when the shape has 256 x 256 tiles
def test_grouped_gemm(F, bn):
    torch.manual_seed(5)
    E, N, K = 4, 384, 256
    rows = [128, 0, 384, 256]  # padded-to-128 expert segments; expert 1 is empty
    block_expert, a_parts = [], []
    for e, r in enumerate(rows):
        block_expert += [e] * (r // 128)
        a_parts.append(torch.randn(r, K, device="cuda", dtype=torch.bfloat16))
    block_expert.append(-1)  # one trailing unused block
    a = torch.cat(a_parts + [torch.zeros(128, K, device="cuda", dtype=torch.bfloat16)])
    w = torch.randn(E * N, K, device="cuda", dtype=torch.bfloat16)
    be = torch.tensor(block_expert, device="cuda", dtype=torch.int32)
    out = torch.zeros(a.shape[0], N, device="cuda", dtype=torch.bfloat16)
    F.gemm(a, w, out=out, block_expert=be, n_per_expert=N, force_bn=bn)
    F.check_kernel_status()
    off = 0
    for e, r in enumerate(rows):
        if r:
            ref = a[off:off + r].float() @ w[e * N:(e + 1) * N].float().t()
            assert _rel_err(out[off:off + r], ref) < 1e-2
        off += r
    assert out[off:].abs().max().item() == 0.0


def test_linear_autograd_matches_reference(F):
    torch.manual_seed(6)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 256, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_()
    y = F.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(w.grad, wr.grad) < 1e-2
    # main_grad convention
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(w2.shape, device="cuda", dtype=torch.float32)
    F.linear(x.detach(), w2).backward(g)
    assert w2.grad is None and _rel_err(w2.main_grad, wr.grad) < 1e-3


def test_router_logits_fp32_accuracy_on_tensor_cores():
    """hi/lo bf16 split of the fp32 router weight (and of the logit gradient): the tcgen05 path must match an fp32 matmul
    far more closely than a plain bf16 cast of the weight would."""
    from paddleformers_b200.ops import functional as F

    torch.manual_seed(0)
    T, H, E = 1000, 512, 128
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(E, H, device="cuda") * 0.05).requires_grad_(True)
    g = torch.randn(T, E, device="cuda")
    out = F.router_logits(x, w)
    out.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    ref = xr @ wr.t()
    ref.backward(g)
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert out.dtype == torch.float32 and rel(out, ref) < 2e-5
    assert rel(w.grad, wr.grad) < 2e-5
    assert rel(x.grad, xr.grad) < 5e-3          # dx is returned in bf16
    F.check_kernel_status()


_REDUCE_WORKER = r'''
import sys, torch
sys.path.insert(0, sys.argv[1])
from paddleformers_b200.ops import functional as F
torch.manual_seed(0)
bad = []
for T, N, K in ((4096, 1024, 512), (2048, 768, 1280), (1000, 512, 264), (4096, 4096, 4096)):
    dy = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    acc = torch.randn(N, K, device="cuda")
    ref = acc.double() + dy.double().t() @ x.double()
    for _ in range(2):                       # two products into the same buffer: the second adds to the first
        F.gemm(dy, x, out=acc, a_mn=True, b_mn=True, epi=F.EPI_ACCUM_F32)
    ref = ref + dy.double().t() @ x.double()
    err = ((acc.double() - ref).norm() / ref.norm()).item()
    if not err < 2e-3:
        bad.append((T, N, K, err))
F.check_kernel_status()
print("RESULT", "OK" if not bad else f"BAD {bad}")
'''


def test_weight_gradient_accumulates_through_tma_reduce_add(tmp_path):
    """The CTA-pair kernel adds its fp32 tiles to the gradient buffer with TMA reduce operations (the sum is formed in L2;
    PFB_GEMM_TMA_REDUCE, on by default). The switch is read once per process, so the check runs in a child process."""
    import os
    import subprocess
    import sys

    script = tmp_path / "w.py"
    script.write_text(_REDUCE_WORKER)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, str(script), repo], env=dict(os.environ, PFB_GEMM_TMA_REDUCE="1"), capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0 and "RESULT OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


_TAIL_WORKER = r'''
import sys, torch
sys.path.insert(0, sys.argv[1])
from paddleformers_b200.ops import functional as F
torch.manual_seed(0)
def rel(a, b): return ((a.double() - b.double()).norm() / b.double().norm()).item()
bad = []
# 256 / 384 tiles of 256 x 256 on 74 CTA pairs: the last round (34 / 14 tiles) is computed as 128-column halves
for M, N, K in ((4096, 4096, 512), (4096, 6144, 256), (4000, 4096, 320)):
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    y = F.gemm(x, w)                                              # forward: both operands K-major
    if not rel(y, x.float() @ w.float().t()) < 6e-3: bad.append(("fwd", M, N, K))
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    dx = F.gemm(dy, w, b_mn=True)                                 # input gradient: B read MN-major
    if not rel(dx, dy.float() @ w.float()) < 6e-3: bad.append(("dgrad", M, N, K))
    acc = torch.randn(N, K, device="cuda")
    ref = acc.double() + dy.double().t() @ x.double()
    F.gemm(dy, x, out=acc, a_mn=True, b_mn=True, epi=F.EPI_ACCUM_F32)    # weight gradient (few tiles here: whole tiles only)
    if not rel(acc, ref) < 2e-3: bad.append(("wgrad", M, N, K))
T, H, I = 4096, 512, 2048
x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
wgu = (torch.randn(2 * I, H, device="cuda") * 0.05).to(torch.bfloat16)
act = F.linear_swiglu(x, wgu) if hasattr(F, "linear_swiglu") else None
if act is not None:
    gu = x.float() @ wgu.float().t()
    if not rel(act, torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]) < 8e-3: bad.append(("swiglu",))
dy = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
xx = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
acc = torch.zeros(4096, 4096, device="cuda")
F.gemm(dy, xx, out=acc, a_mn=True, b_mn=True, epi=F.EPI_ACCUM_F32)       # 256 tiles: split tail with the accumulate epilogue
if not rel(acc, dy.float().t() @ xx.float()) < 2e-3: bad.append(("wgrad_tail",))
F.check_kernel_status()
print("RESULT", "OK" if not bad else f"BAD {bad}")
'''


@pytest.mark.parametrize("env", [dict(PFB_GEMM_TAIL_SPLIT="1", PFB_GEMM_TMA_REDUCE="0"), dict(PFB_GEMM_TAIL_SPLIT="1", PFB_GEMM_TMA_REDUCE="1"),
                                 dict(PFB_GEMM_TAIL_SPLIT="0", PFB_GEMM_TMA_REDUCE="0")])
def test_last_round_of_tiles_split_into_half_tiles(tmp_path, env):
    """Tiles of the last, partly filled round are computed as two 128-column halves (PFB_GEMM_TAIL_SPLIT, on by default);
    every epilogue and operand layout against fp32, with the switches on and off (they are read once per process, so the
    check runs in a child process)."""
    import os
    import subprocess
    import sys

    script = tmp_path / "w.py"
    script.write_text(_TAIL_WORKER)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, str(script), repo], env=dict(os.environ, **env), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "RESULT OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
