"""A device-side wait that nothing satisfies must run out, leave an error code in the status word and return, and the
next kernel must work: the failure-detection path of the peer-memory kernels, exercised on ONE GPU by handing a kernel
flags that no peer ever raises (no rank is killed, nothing faults)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

PFB_ERR_WAIT_PEER = 5


@pytest.fixture()
def F():
    from paddleformers_b200.ops import functional as F

    F.check_kernel_status()
    yield F
    torch.ops.pfb200.set_wait_budget(0.0)     # back to the default budget
    torch.ops.pfb200.read_status(True)


def test_flag_wait_runs_out_and_reports(F):
    from paddleformers_b200.parallel.symmetric_memory import FlagPad

    pad = FlagPad(8, None)
    pad.wait(0, 1, value=1, timeout_s=0.005)           # flag 0 is never raised
    assert int(torch.ops.pfb200.read_status(True)) == PFB_ERR_WAIT_PEER
    a = torch.randn(256, 256, device="cuda", dtype=torch.bfloat16)
    out = F.gemm(a, a)
    assert int(torch.ops.pfb200.read_status(True)) == 0
    assert torch.isfinite(out.float()).all()


def test_all_gather_gemm_gives_up_when_the_peer_never_arrives(F):
    """Rank 0 of a two-rank all-gather GEMM whose peer never launches: the copy CTAs wait for the peer's ready flag, the
    GEMM CTAs for the block flags; with a 2 ms budget every CTA gives up, the kernel returns and reports the wait."""
    from paddleformers_b200.parallel.symmetric_memory import SymmetricBuffer

    T, K, N = 512, 256, 256
    g0, g1 = SymmetricBuffer(T * K * 2, None), SymmetricBuffer(T * K * 2, None)     # "rank 1" is just another local buffer
    r0, r1 = SymmetricBuffer(64, None), SymmetricBuffer(64, None)
    G = g0.tensor((T, K), torch.bfloat16)
    G.normal_()
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
    blk = torch.zeros(T // 128, dtype=torch.int32, device="cuda")
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")
    torch.ops.pfb200.set_wait_budget(0.002)
    torch.ops.pfb200.ag_gemm(G, torch.tensor([g0.local_ptr, g1.local_ptr], dtype=torch.int64), w, out, None, F.EPI_STORE_BF16, False,
                             r0.local_ptr, torch.tensor([r0.local_ptr, r1.local_ptr], dtype=torch.int64), blk, epoch, 0, 2, 2)
    assert int(torch.ops.pfb200.read_status(True)) == PFB_ERR_WAIT_PEER
    torch.ops.pfb200.set_wait_budget(0.0)
    ref = F.gemm(G[:128].contiguous(), w)              # the device and the library are still usable
    assert int(torch.ops.pfb200.read_status(True)) == 0
    assert torch.isfinite(ref.float()).all()


def test_expert_exchange_wait_gives_up(F):
    """``ep_wait_flag`` on a two-rank table whose second rank never signals."""
    from paddleformers_b200.parallel.symmetric_memory import SymmetricBuffer

    ep, EL = 2, 4
    n = 2 * ep * EL + 8 * 8
    t0, t1 = SymmetricBuffer(n * 4, None), SymmetricBuffer(n * 4, None)
    ptrs = torch.tensor([t0.local_ptr, t1.local_ptr], dtype=torch.int64)
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")
    torch.ops.pfb200.set_wait_budget(0.002)
    torch.ops.pfb200.ep_wait_flag(ptrs, 0, ep, EL, 2, epoch)
    assert int(torch.ops.pfb200.read_status(True)) == PFB_ERR_WAIT_PEER
