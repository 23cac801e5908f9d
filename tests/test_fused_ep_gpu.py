"""Peer-memory expert-parallel dispatch / combine kernels against the NCCL all-to-all path.

The worker runs as child processes, one per GPU (NVLS off; the kernels use plain peer loads and stores). With one GPU
the expert-parallel group has a single rank and the same kernels exchange with themselves, which covers the slot
arithmetic, the flags and the autograd wiring."""
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
from paddleformers_b200.parallel import fused_ep
from paddleformers_b200.parallel.expert_parallel import _alltoall_moe_forward
from paddleformers_b200.models.configuration import Qwen3MoeConfig
from paddleformers_b200.nn.moe import MoELayer, build_dispatch_plan, _PermuteFn, unpermute_combine
from paddleformers_b200.ops import functional as F

world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
ps = initialize_parallel(ParallelDegrees(sharding=world, ep=world))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
torch.manual_seed(11 + ps.rank_in("ep"))
T, H, E, k, I = 512, 256, 8, 4, 128
cfg = Qwen3MoeConfig(hidden_size=H, num_experts=E, num_experts_per_tok=k, moe_intermediate_size=I, intermediate_size=I,
                     num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, vocab_size=64)
layers = [MoELayer(cfg, dtype=torch.bfloat16, device=dev) for _ in range(2)]
for l in layers:
    for p_ in l.parameters():
        torch.nn.init.normal_(p_, std=0.05)
def rel(a, b): return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()
errs = {}
for it in range(3):          # several exchanges: epochs advance, the shared gradient buffers are reused across layers
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    routing = []
    for l in layers:
        idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)])
        if it == 2:
            idx[:, 0] = 0    # skewed: expert 0 receives every token (stays inside the 1.5x capacity for these sizes)
            idx[:, 1:] = torch.stack([1 + torch.randperm(E - 1, device=dev)[:k - 1] for _ in range(T)])
        w = torch.rand(T, k, device=dev, dtype=torch.float32).requires_grad_(True)
        routing.append((idx, w))
    outs = {}
    for mode in ("fused", "nccl"):
        for p_ in [x] + [p_ for l in layers for p_ in l.parameters()] + [w for _, w in routing]:
            p_.grad = None
        h = x
        for l, (idx, w) in zip(layers, routing):
            if mode == "fused":
                ws = fused_ep.get_workspace(ps, h, l)
                h = h + fused_ep.moe_forward(ws, l, h, idx, w)
            elif world > 1:
                h = h + _alltoall_moe_forward(l, h, idx, w, ps)
            else:            # one rank: the local permutation path is the reference
                dest, block_expert, rows, counts = build_dispatch_plan(idx, E, 0)
                yr = l.experts(_PermuteFn.apply(h, dest, k, rows), block_expert, counts)
                h = h + unpermute_combine(yr, dest, w, T).to(h.dtype)
        h.backward(g)
        outs[mode] = [t.detach().clone() for t in [h, x.grad] + [w.grad for _, w in routing]
                      + [l.experts.gate_up_proj.grad for l in layers] + [l.experts.down_proj.grad for l in layers]]
    F.check_kernel_status()
    names = ["y", "dx", "dw0", "dw1", "dgu0", "dgu1", "ddn0", "ddn1"]
    for name, a, b in zip(names, outs["fused"], outs["nccl"]):
        errs[f"{it}_{name}"] = rel(a, b)
bad = {k_: v for k_, v in errs.items() if not v < 3e-2}
print("RESULT", "OK" if not bad else f"BAD {bad}", "calls", fused_ep.STATS, flush=True)
if dist.is_initialized():
    dist.barrier(); dist.destroy_process_group()
'''


def _run(tmp_path, nproc, port):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PFB_REPO=repo)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr=127.0.0.1",
           f"--master-port={port}", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    # the ranks write into one pipe at the same time, so two of their lines can interleave: count tokens, not lines
    assert res.stdout.count("OK") >= nproc and res.stdout.count("RESULT") == nproc and "BAD" not in res.stdout, res.stdout[-3000:]


def test_fused_ep_single_rank(tmp_path):
    _run(tmp_path, 1, 29551)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_ep_matches_alltoall_two_ranks(tmp_path):
    _run(tmp_path, 2, 29552)


def test_guard_words_behind_peer_memory_regions_catch_an_overrun(monkeypatch):
    """PFB_DEBUG_CANARY=1 places 1 KB of guard words behind every region of a symmetric arena; a write past a region's end
    (here made through a wider view of the same allocation, so nothing leaves the buffer) is reported."""
    from paddleformers_b200.parallel import fused_collectives as fc

    monkeypatch.setenv("PFB_DEBUG_CANARY", "1")
    arena = fc.SymmetricArena(None)
    a = fc._Region(arena, (300,), torch.float32)          # 1200 bytes -> payload rounded to 2048, guard behind it
    b = fc._Region(arena, (64, 8), torch.bfloat16)
    a.tensor.fill_(1.0)
    b.tensor.fill_(2.0)
    assert fc.check_canaries() == 0
    buf = arena.chunks[0]
    wide = buf.tensor((2048 // 4 + 4,), torch.float32, a.local_ptr - buf.local_ptr)
    wide[2048 // 4 + 1] = 7.0                              # one word into a's guard
    assert fc.check_canaries() == 1
    fc._CANARIES.clear()
    for ch in arena.chunks:
        ch.close()
