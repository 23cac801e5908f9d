"""Fused all-gather-GEMM / GEMM-reduce-scatter kernels against the NCCL + GEMM path on 2 GPUs (child processes,
NVLS off, plain peer loads / stores)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["PFB_REPO"])
from paddleformers_b200.parallel.topology import ParallelDegrees, initialize_parallel
from paddleformers_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
from paddleformers_b200.ops import functional as F

ps = initialize_parallel(ParallelDegrees(mp=int(os.environ["WORLD_SIZE"])))
tp, rank = ps.degrees.mp, ps.coord["mp"]
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
torch.manual_seed(7)
T, H, I = 1024, 512, 1024
def rel(a, b): return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()
errs = {}
for it in range(3):   # several calls: exercises epochs and the alternating staging buffers
    col = ColumnParallelLinear(H, 2 * I, sections=[I, I], sequence_parallel=True, epilogue="swiglu", dtype=torch.bfloat16, device=dev)
    row = RowParallelLinear(I, H, sequence_parallel=True, dtype=torch.bfloat16, device=dev)
    torch.nn.init.normal_(col.weight, std=0.05); torch.nn.init.normal_(row.weight, std=0.05)
    x = torch.randn(T // tp, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(T // tp, H, device=dev, dtype=torch.bfloat16)
    outs = {}
    for mode in ("1", "0"):
        os.environ["PFB_FUSED_TP"] = mode
        for p_ in (x, col.weight, row.weight): p_.grad = None
        y = row(col(x))
        y.backward(g)
        outs[mode] = [t.detach().clone() for t in (y, x.grad, col.weight.grad, row.weight.grad)]
    F.check_kernel_status()
    for name, a, b in zip(("y", "dx", "dw_col", "dw_row"), outs["1"], outs["0"]):
        errs[f"{it}_{name}"] = rel(a, b)
bad = {k: v for k, v in errs.items() if not v < 2e-2}
print("RESULT", "OK" if not bad else f"BAD {bad}", flush=True)
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp_linears_match_nccl_path(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PFB_REPO=repo)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr=127.0.0.1",
           "--master-port=29541", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("RESULT")]
    assert len(lines) == 2 and all(l == "RESULT OK" for l in lines), res.stdout[-3000:]
