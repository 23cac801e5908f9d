"""Optimizer sharding through the peer-memory kernels (reduce + scale + norm in one pass, AdamW whose bf16 output is the
all-gather) against the NCCL reduce-scatter / all-gather path, on 2 GPUs (child processes, NVLS off). With two ranks the
sum a + b has one order, so the two paths must agree bit for bit."""
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
from paddleformers_b200.parallel.sharding import ShardedAdamW
from paddleformers_b200.models.configuration import named_config
from paddleformers_b200.transformers.auto import AutoModelForCausalLM
from paddleformers_b200.ops import functional as F

world = int(os.environ["WORLD_SIZE"])
ps = initialize_parallel(ParallelDegrees(sharding=world))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
rank = dist.get_rank()

def run(fused):
    os.environ["PFB_FUSED_SHARDING"] = "1" if fused else "0"
    torch.manual_seed(5)
    cfg = named_config("tiny-llama", num_hidden_layers=2)
    cfg.dtype = "bfloat16"
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16, device=dev)
    opt = ShardedAdamW(model, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0, parallel_state=ps)
    assert (opt.domains[0].symm is not None) == fused
    g = torch.Generator().manual_seed(100 + rank)           # different data per rank: the reduction matters
    norms = []
    for step in range(3):
        ids = torch.randint(0, cfg.vocab_size, (2, 128), generator=g).to(dev)
        out = model(input_ids=ids, labels=ids)
        out.loss.backward()
        opt.accumulate_grads()
        norms.append(float(opt.step()))
    F.check_kernel_status()
    flat = torch.cat([d.flat_param.float().clone() for d in opt.domains])
    return flat, norms

a, na = run(True)
b, nb = run(False)
same = torch.equal(a, b)
# every rank must hold the same parameters after the push
ref = a.clone(); dist.broadcast(ref, 0)
agree = torch.equal(ref, a)
print("RESULT", "OK" if (same and agree and na == nb) else f"BAD same={same} agree={agree} norms={na} vs {nb}", flush=True)
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_sharding_matches_nccl_path_bitwise(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PFB_REPO=repo)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr=127.0.0.1",
           "--master-port=29547", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    # the ranks write into one pipe at the same time, so two of their lines can interleave: count tokens, not lines
    assert res.stdout.count("OK") >= 2 and res.stdout.count("RESULT") == 2 and "BAD" not in res.stdout, res.stdout[-3000:]
