"""Parallel strategies on 2 GPUs (NCCL, bf16, the CUDA kernels): pipeline schedules, ZeRO-3, context / ring / Ulysses
attention and the peer-memory expert exchange must reproduce the single-GPU losses of the same weights and data.

One child job computes the single-GPU reference, a second one (2 ranks) runs every strategy in turn; NVLS is off and
ranks leave only after a barrier."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

_WORKER = r'''
import json, os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["PFB_REPO"])
from paddleformers_b200 import Trainer, TrainingArguments
from paddleformers_b200.models.configuration import named_config
from paddleformers_b200.models.modeling import MODEL_MAPPING
from paddleformers_b200.parallel.pipeline import build_pipeline_model
from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
from paddleformers_b200.transformers.model_utils import param_shard_spec
from paddleformers_b200.ops import functional as F

world = int(os.environ["WORLD_SIZE"]); rank = int(os.environ["RANK"])
ON_GPU = os.environ.get("PFB_TEST_DEVICE", "cuda") == "cuda"       # "cpu": dry run of the same script on gloo ranks in fp32
if ON_GPU:
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"])); torch.cuda.set_device(dev)
else:
    dev = torch.device("cpu")
DT = torch.bfloat16 if ON_GPU else torch.float32
S, STEPS, V = 256, 2, 512

def cfg_for(moe, layers):
    if moe:
        return named_config("qwen3-30b-a3b", num_hidden_layers=layers, hidden_size=256, num_attention_heads=2, num_key_value_heads=2,
                            head_dim=128, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=128, vocab_size=V,
                            router_aux_loss_coef=0.0)
    return named_config("tiny-llama", num_hidden_layers=layers, hidden_size=256, intermediate_size=512, num_attention_heads=2,
                        num_key_value_heads=2, head_dim=128, vocab_size=V)

def data(n):
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, V, (n, S + 1), generator=g)
    labels = ids[:, 1:].clone(); labels[:, :3] = -100
    return [{"input_ids": ids[i, :-1], "labels": labels[i]} for i in range(n)]

class DS(torch.utils.data.Dataset):
    def __init__(self, items): self.items = items
    def __len__(self): return len(self.items)
    def __getitem__(self, i): return self.items[i]

def full_weights(moe, layers):
    torch.manual_seed(5)
    cfg = cfg_for(moe, layers)
    m = MODEL_MAPPING[cfg.model_type](cfg)
    return {k: v.detach().clone() for k, v in m.named_parameters()}

def train(moe, layers, pipeline, targs):
    targs = dict(targs)
    os.environ.update(targs.pop("_env", {}))
    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=1, max_steps=STEPS, learning_rate=1e-3,
                             lr_scheduler_type="constant", logging_steps=1, save_strategy="no", max_seq_len=S, max_grad_norm=1.0,
                             seed=3, bf16=ON_GPU, device=str(dev), **targs)
    ps = args.setup_parallel()
    cfg = cfg_for(moe, layers)
    cfg.dtype = "bfloat16" if ON_GPU else "float32"
    LlmMetaConfig.set_llm_config(cfg, args)
    full = FULL[(moe, layers)]
    if pipeline:
        model = build_pipeline_model(cfg, dtype=DT, device=dev)
    else:
        model = MODEL_MAPPING[cfg.model_type].from_config(cfg, dtype=DT, device=dev)
    with torch.no_grad():
        for name, p in model.named_parameters():
            g = model.global_param_name(name) if pipeline else name
            spec = param_shard_spec(p)
            p.copy_(spec.shard(full[g], ps.coord["mp"], ps.degrees.mp, ps.rank_in("ep"), ps.degrees.ep).to(device=dev, dtype=p.dtype))
    tr = Trainer(model=model, args=args, train_dataset=DS(data(8 * STEPS)))
    tr._sampler_shuffle = False
    tr.train()
    if ON_GPU:
        F.check_kernel_status()
    return [h["loss"] for h in tr.state.log_history if "loss" in h]

CASES = json.loads(os.environ["PFB_CASES"])
# the full (unsharded) weights are drawn before any parallel topology exists, so that every case cuts the same tensors
FULL = {(moe, layers): full_weights(moe, layers) for moe, layers in {(c[0], c[1]) for c in CASES.values()}}
out = {}
for name, (moe, layers, pipeline, targs) in CASES.items():
    out[name] = train(moe, layers, pipeline, targs)
    if dist.is_initialized(): dist.barrier()
if rank == 0:
    from paddleformers_b200.parallel import fused_ep
    out["_fused_ep_dispatches"] = fused_ep.STATS["dispatch"]
    json.dump(out, open(os.environ["PFB_OUT"], "w"))
if dist.is_initialized():
    dist.barrier(); dist.destroy_process_group()
print("RESULT OK", flush=True)
'''


def _launch(tmp_path, n, cases, out, port):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PFB_REPO=repo, PFB_CASES=json.dumps(cases), PFB_OUT=str(out))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr=127.0.0.1",
           f"--master-port={port}", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return json.load(open(out))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_parallel_strategies_match_single_gpu(tmp_path):
    acc4 = dict(gradient_accumulation_steps=4)
    ref = _launch(tmp_path, 1, {
        "dense2": (False, 2, False, dict(gradient_accumulation_steps=2)),
        "dense4": (False, 4, False, acc4),
        "moe2": (True, 2, False, dict(gradient_accumulation_steps=2, moe_token_dispatcher_type="alltoall")),
    }, tmp_path / "ref.json", 29571)
    cases = {
        "pp2_1f1b": (False, 4, True, dict(pipeline_model_parallel_size=2, **acc4)),
        "pp2_zero_bubble": (False, 4, True, dict(pipeline_model_parallel_size=2, pipeline_schedule="zero_bubble", **acc4)),
        "pp2_interleaved": (False, 4, True, dict(pipeline_model_parallel_size=2, virtual_pipeline_model_parallel_size=2,
                                                 pipeline_schedule="interleaved", **acc4)),
        "stage3_fsdp2": (False, 2, False, dict(sharding="stage3", gradient_accumulation_steps=1)),
        "sharding2_stage1": (False, 2, False, dict(sharding="stage1", gradient_accumulation_steps=1)),
        "cp2": (False, 2, False, dict(context_parallel_size=2, gradient_accumulation_steps=2)),
        "cp2_ring": (False, 2, False, dict(context_parallel_size=2, context_parallel_algo="ring", gradient_accumulation_steps=2)),
        "sep2": (False, 2, False, dict(sep_parallel_size=2, gradient_accumulation_steps=2)),
        "ep2_fused": (True, 2, False, dict(expert_model_parallel_size=2, sharding="stage1", gradient_accumulation_steps=1,
                                           moe_token_dispatcher_type="fused")),
    }
    got = _launch(tmp_path, 2, cases, tmp_path / "got.json", 29572)
    base = {"pp2": "dense4", "ep2": "moe2"}
    bad = {}
    got.pop("_fused_ep_dispatches", None)
    for name, losses in got.items():
        want = ref[base.get(name[:3], "dense2")]
        for a, b in zip(want, losses):
            if not abs(a - b) < 3e-2 * max(1.0, abs(a)):        # bf16 forward and backward, different reduction orders
                bad[name] = (want, losses)
    assert not bad, bad


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_pipeline_stages_use_the_peer_memory_expert_exchange(tmp_path):
    """Several micro-batches are in flight per pipeline stage: the exchange keeps one buffer slot per micro-batch. With two
    GPUs both are pipeline stages, so each stage's expert-parallel group has one rank and PFB_FUSED_EP_SINGLE sends it
    through the exchange kernels all the same."""
    acc4 = dict(gradient_accumulation_steps=4)
    ref = _launch(tmp_path, 1, {"moe4": (True, 4, False, dict(moe_token_dispatcher_type="alltoall", **acc4))},
                  tmp_path / "ref.json", 29573)
    got = _launch(tmp_path, 2, {
        "pp2_moe_fused_1f1b": (True, 4, True, dict(pipeline_model_parallel_size=2, moe_token_dispatcher_type="fused",
                                                   _env={"PFB_FUSED_EP_SINGLE": "1"}, **acc4)),
        "pp2_moe_fused_interleaved": (True, 4, True, dict(pipeline_model_parallel_size=2, virtual_pipeline_model_parallel_size=2,
                                                          pipeline_schedule="interleaved", moe_token_dispatcher_type="fused",
                                                          _env={"PFB_FUSED_EP_SINGLE": "1"}, **acc4)),
    }, tmp_path / "got.json", 29574)
    for name, losses in got.items():
        if name.startswith("_"):
            continue
        for a, b in zip(ref["moe4"], losses):
            assert abs(a - b) < 3e-2 * max(1.0, abs(a)), (name, ref["moe4"], losses)
    assert got["_fused_ep_dispatches"] > 0, got
