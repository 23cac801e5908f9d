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



_WORKER_FP32 = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["PFB_REPO"])
from paddleformers_b200.parallel.topology import ParallelDegrees, initialize_parallel
from paddleformers_b200.parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
from paddleformers_b200.ops import functional as F

# The tensor-parallel linears of one Llama-3-8B layer at the benchmark's shapes (T 4096, hidden 4096, ffn 14336, qkv 6144;
# per-rank widths 768 / 3584 and depths 512 / 1792 at 8 ranks) against the same layer computed whole in fp32.
torch.backends.cuda.matmul.allow_tf32 = False
ps = initialize_parallel(ParallelDegrees(mp=int(os.environ["WORLD_SIZE"])))
tp, rank = ps.degrees.mp, ps.coord["mp"]
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
T, H, I, QKV = 4096, 4096, 14336, 6144
R = T // tp
def rel(a, b): return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()
g = torch.Generator(device=dev).manual_seed(11)      # the same full tensors on every rank
x_full = torch.randn(T, H, device=dev, generator=g).bfloat16()
w_qkv = (torch.randn(QKV, H, device=dev, generator=g) * 0.02).bfloat16()
w_o = (torch.randn(H, QKV, device=dev, generator=g) * 0.02).bfloat16()
w_gu = (torch.randn(2 * I, H, device=dev, generator=g) * 0.02).bfloat16()
w_d = (torch.randn(H, I, device=dev, generator=g) * 0.02).bfloat16()
gy = torch.randn(T, H, device=dev, generator=g).bfloat16()
errs = {}
os.environ["PFB_FUSED_TP"] = "1"
for it in range(2):
    # ---- "attention-like" pair: qkv projection (column parallel) then a row-parallel projection of its output
    col = ColumnParallelLinear(H, QKV, sequence_parallel=True, dtype=torch.bfloat16, device=dev)
    row = RowParallelLinear(QKV, H, sequence_parallel=True, dtype=torch.bfloat16, device=dev)
    n = QKV // tp
    with torch.no_grad():
        col.weight.copy_(w_qkv[rank * n:(rank + 1) * n]); row.weight.copy_(w_o[:, rank * n:(rank + 1) * n])
    x = x_full[rank * R:(rank + 1) * R].clone().requires_grad_()
    y = row(col(x)); y.backward(gy[rank * R:(rank + 1) * R])
    xr = x_full.float().requires_grad_(); wq = w_qkv.float().requires_grad_(); wo = w_o.float().requires_grad_()
    mid = (xr @ wq.t()).bfloat16().float()              # the fused path rounds the intermediate to bf16 too
    yr = mid @ wo.t(); yr.backward(gy.float())
    errs[f"{it}_attn_y"] = rel(y, yr[rank * R:(rank + 1) * R]); errs[f"{it}_attn_dx"] = rel(x.grad, xr.grad[rank * R:(rank + 1) * R])
    errs[f"{it}_attn_dwcol"] = rel(col.weight.main_grad if hasattr(col.weight, "main_grad") else col.weight.grad, wq.grad[rank * n:(rank + 1) * n])
    errs[f"{it}_attn_dwrow"] = rel(row.weight.main_grad if hasattr(row.weight, "main_grad") else row.weight.grad, wo.grad[:, rank * n:(rank + 1) * n])
    del col, row, xr, wq, wo, mid, yr
    # ---- MLP pair: gate_up with the SwiGLU epilogue (column parallel) then down (row parallel)
    col = ColumnParallelLinear(H, 2 * I, sections=[I, I], sequence_parallel=True, epilogue="swiglu", dtype=torch.bfloat16, device=dev)
    row = RowParallelLinear(I, H, sequence_parallel=True, dtype=torch.bfloat16, device=dev)
    m = I // tp
    with torch.no_grad():
        col.weight[:m].copy_(w_gu[rank * m:(rank + 1) * m]); col.weight[m:].copy_(w_gu[I + rank * m:I + (rank + 1) * m])
        row.weight.copy_(w_d[:, rank * m:(rank + 1) * m])
    x = x_full[rank * R:(rank + 1) * R].clone().requires_grad_()
    y = row(col(x)); y.backward(gy[rank * R:(rank + 1) * R])
    xr = x_full.float().requires_grad_(); wgu = w_gu.float().requires_grad_(); wd = w_d.float().requires_grad_()
    gu = xr @ wgu.t()
    act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    yr = act @ wd.t(); yr.backward(gy.float())
    errs[f"{it}_mlp_y"] = rel(y, yr[rank * R:(rank + 1) * R]); errs[f"{it}_mlp_dx"] = rel(x.grad, xr.grad[rank * R:(rank + 1) * R])
    gcol = col.weight.main_grad if hasattr(col.weight, "main_grad") else col.weight.grad
    errs[f"{it}_mlp_dwgate"] = rel(gcol[:m], wgu.grad[rank * m:(rank + 1) * m])
    errs[f"{it}_mlp_dwup"] = rel(gcol[m:], wgu.grad[I + rank * m:I + (rank + 1) * m])
    errs[f"{it}_mlp_dwdown"] = rel(row.weight.main_grad if hasattr(row.weight, "main_grad") else row.weight.grad, wd.grad[:, rank * m:(rank + 1) * m])
    del col, row, xr, wgu, wd, gu, act, yr
    F.check_kernel_status()
bad = {k: round(v, 4) for k, v in errs.items() if not v < 2e-2}
print("RESULT", "OK" if not bad else f"BAD {bad}", flush=True)
dist.barrier(); dist.destroy_process_group()
"""


def _run_workers(tmp_path, text, n, port):
    script = tmp_path / "worker.py"
    script.write_text(text)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PFB_REPO=repo)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr=127.0.0.1",
           f"--master-port={port}", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    # the ranks write into one pipe at the same time, so two of their lines can interleave: count tokens, not lines
    assert res.stdout.count("OK") >= n and res.stdout.count("RESULT") == n and "BAD" not in res.stdout, res.stdout[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp_linears_match_fp32_at_benchmark_shapes_2_ranks(tmp_path):
    _run_workers(tmp_path, _WORKER_FP32, 2, 29543)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_fused_tp_linears_match_fp32_at_benchmark_shapes_8_ranks(tmp_path):
    _run_workers(tmp_path, _WORKER_FP32, 8, 29544)


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
    # the ranks write into one pipe at the same time, so two of their lines can interleave: count tokens, not lines
    assert res.stdout.count("OK") >= 2 and res.stdout.count("RESULT") == 2 and "BAD" not in res.stdout, res.stdout[-3000:]
