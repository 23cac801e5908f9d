"""Optimizer variants over the flat sharded buffers: bit-exact agreement with torch.optim.AdamW, low-precision and
host-resident moments, one-second-moment-per-row AdamW."""
import copy

import pytest
import torch

from paddleformers_b200.parallel.sharding import ShardedAdamW
from paddleformers_b200.parallel.topology import ParallelDegrees, ParallelState, set_parallel_state
from paddleformers_b200.utils.optimizer import AdamWCustom, AdamWMini


class _Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a = torch.nn.Linear(24, 40)
        self.norm = torch.nn.LayerNorm(40)
        self.b = torch.nn.Linear(40, 8, bias=False)

    def forward(self, x):
        return self.b(self.norm(torch.tanh(self.a(x))))


def _state():
    ps = ParallelState(ParallelDegrees(), rank=0, create_groups=False)
    set_parallel_state(ps)
    return ps


def _run(opt_factory, steps=6, seed=0):
    torch.manual_seed(seed)
    net = _Net()
    opt = opt_factory(net)
    torch.manual_seed(seed + 1)
    for _ in range(steps):
        x = torch.randn(16, 24)
        net(x).pow(2).mean().backward()
        opt.step()
    return net, opt


@pytest.mark.parametrize("clip", [0.0, 0.05])
def test_bitexact_mode_reproduces_torch_adamw_bit_for_bit(clip):
    ps = _state()
    kw = dict(lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    net, _ = _run(lambda m: AdamWCustom(m, max_grad_norm=clip, parallel_state=ps, hf_bitexact=True, **kw))
    # the same run with torch: decay rule by name (bias / norm not decayed), clip_grad_norm_, optimizer.step
    torch.manual_seed(0)
    ref = _Net()
    decay = [p for n, p in ref.named_parameters() if not ("bias" in n or "norm" in n)]
    rest = [p for n, p in ref.named_parameters() if ("bias" in n or "norm" in n)]
    topt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}],
                             lr=3e-3, betas=(0.9, 0.95), eps=1e-8, foreach=False)
    torch.manual_seed(1)
    for _ in range(6):
        x = torch.randn(16, 24)
        ref(x).pow(2).mean().backward()
        if clip:
            torch.nn.utils.clip_grad_norm_(ref.parameters(), clip, foreach=False)
        topt.step()
        topt.zero_grad()
    for (n, p), (_, q) in zip(net.named_parameters(), ref.named_parameters()):
        assert torch.equal(p, q), n
    # the default update order is close but not identical in bits
    net2, _ = _run(lambda m: ShardedAdamW(m, max_grad_norm=clip, parallel_state=ps, **kw))
    assert all(torch.allclose(p, q, rtol=1e-4, atol=1e-6) for p, q in zip(net2.parameters(), ref.parameters()))


def test_bf16_and_host_resident_moments_track_the_fp32_optimizer():
    ps = _state()
    kw = dict(lr=3e-3, weight_decay=0.01, max_grad_norm=1.0, parallel_state=ps)
    base, bopt = _run(lambda m: ShardedAdamW(m, **kw))
    # chunked streaming of fp32 moments changes nothing
    off, oopt = _run(lambda m: AdamWCustom(m, offload_moments=True, offload_chunk_numel=100, **kw))
    for p, q in zip(base.parameters(), off.parameters()):
        assert torch.allclose(p, q, rtol=1e-6, atol=1e-7)
    assert all(d.exp_avg.device.type == "cpu" for d in oopt.domains)
    # bf16 moments: same trajectory within the rounding of the moments
    low, lopt = _run(lambda m: AdamWCustom(m, moment_dtype=torch.bfloat16, **kw))
    assert all(d.exp_avg.dtype == torch.bfloat16 and d.exp_avg_sq.dtype == torch.bfloat16 for d in lopt.domains)
    err = max(float((p - q).abs().max()) for p, q in zip(base.parameters(), low.parameters()))
    moved = max(float((p - q).abs().max()) for p, q in zip(base.parameters(), _Net().parameters()))
    assert err < 2e-3 and err < 0.2 * moved
    # state round trip keeps the dtype
    sd = copy.deepcopy(lopt.state_dict())
    _, fresh = _run(lambda m: AdamWCustom(m, moment_dtype=torch.bfloat16, **kw), steps=0)
    fresh.load_state_dict(sd)
    assert all(torch.equal(a.exp_avg, b.exp_avg) and torch.equal(a.master, b.master) for a, b in zip(fresh.domains, lopt.domains))


def test_adamw_mini_keeps_one_second_moment_per_row_and_trains():
    ps = _state()
    torch.manual_seed(0)
    net = _Net()
    opt = AdamWMini(net, lr=1e-2, weight_decay=0.0, max_grad_norm=0.0, parallel_state=ps)
    n_elems = sum(p.numel() for p in net.parameters())
    # rows: a.weight 40, b.weight 8; vectors: a.bias, norm.weight, norm.bias; plus alignment-padding blocks
    real_blocks = 40 + 8 + 3
    assert real_blocks <= opt.second_moment_numel() <= real_blocks + 2 * 5 and opt.second_moment_numel() < n_elems // 10
    # first step: every element of a row moves by lr * g / (|g|_rms of the row) (bias corrections cancel)
    before = {n: p.detach().clone() for n, p in net.named_parameters()}
    x = torch.randn(16, 24)
    net(x).pow(2).mean().backward()
    g = net.a.weight.grad.clone()
    opt.step()
    want = before["a.weight"] - 1e-2 * g / (g.pow(2).mean(-1, keepdim=True).sqrt() + 1e-8)
    assert torch.allclose(net.a.weight, want, rtol=1e-5, atol=1e-7)
    losses = []
    torch.manual_seed(1)
    xs = torch.randn(64, 24)
    for _ in range(30):
        loss = net(xs).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < 0.5 * losses[0]


def test_trainer_selects_optimizer_variants(tmp_path):
    from paddleformers_b200 import AutoModelForCausalLM, Trainer, TrainingArguments
    from paddleformers_b200.data.synthetic import SyntheticCausalLMDataset
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.trainer.trainer_utils import OptimizerNames

    assert {o.value for o in OptimizerNames} == {"adamw", "adamw_mini", "adamw_custom", "muon"}
    for kw, cls in ((dict(optim="adamw_mini"), AdamWMini), (dict(use_lowprecision_moment=True), AdamWCustom),
                    (dict(optim="adamw_custom", hf_bitexact=True), AdamWCustom)):
        torch.manual_seed(0)
        model = AutoModelForCausalLM.from_config(named_config("tiny-llama", vocab_size=128))
        args = TrainingArguments(output_dir=str(tmp_path), per_device_train_batch_size=2, max_steps=3, learning_rate=1e-3,
                                 save_strategy="no", max_seq_len=32, lr_scheduler_type="constant", **kw)
        tr = Trainer(model=model, args=args, train_dataset=SyntheticCausalLMDataset(128, 32, 16, seed=0))
        tr.train()
        assert type(tr.optimizer) is cls
        losses = [h["loss"] for h in tr.state.log_history if "loss" in h]
        assert len(losses) == 3 and all(l == l for l in losses)


def test_stage3_units_share_one_working_buffer_and_match_the_flat_optimizer():
    """One process: per-layer units with recompute reproduce the flat optimizer's trajectory on a MoE model; layer parameters
    are views of ONE buffer of the size of the largest layer; evaluation without a graph gathers too."""
    from paddleformers_b200.models.configuration import Qwen3MoeConfig
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.parallel.fsdp import FullyShardedOptimizer

    ps = _state()
    cfg = Qwen3MoeConfig(vocab_size=96, hidden_size=32, intermediate_size=48, moe_intermediate_size=16, num_hidden_layers=3,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=8, num_experts=4, num_experts_per_tok=2,
                         router_aux_loss_coef=0.01, mlp_only_layers=[1])
    kw = dict(lr=5e-3, weight_decay=0.1, max_grad_norm=1.0, parallel_state=ps)

    def run(make):
        torch.manual_seed(0)
        model = MODEL_MAPPING[cfg.model_type](cfg).float().train()
        opt = make(model)
        g = torch.Generator().manual_seed(1)
        losses = []
        for _ in range(3):
            for _ in range(2):                                   # two micro-batches per step
                ids = torch.randint(0, 96, (2, 12), generator=g)
                out = model(ids, labels=torch.roll(ids, -1, 1))
                out.loss.backward()
                opt.accumulate_grads()
                losses.append(float(out.loss))
            opt.step()
        return model, opt, losses

    base, bopt, l0 = run(lambda m: ShardedAdamW(m, **kw))
    s3m, s3, l1 = run(lambda m: FullyShardedOptimizer(m, **kw))
    assert l0 == pytest.approx(l1, rel=1e-5, abs=1e-6)
    ref = dict(base.named_parameters())
    for n, p in s3m.named_parameters():
        torch.testing.assert_close(s3.full_tensor(p), ref[n].detach(), rtol=1e-5, atol=1e-6, msg=n)
    assert len(s3.units) == 3 and s3.root is not None
    biggest = max(u.numel for u in s3.units)
    assert s3._pbuf.numel() == biggest
    ptrs = {p.data_ptr() for u in s3.units for _, p in u.params}
    lo, hi = s3._pbuf.data_ptr(), s3._pbuf.data_ptr() + biggest * s3._pbuf.element_size()
    assert all(lo <= x < hi for x in ptrs)
    # without a graph (evaluation, generation) the layers gather their parameters as well
    ids = torch.randint(0, 96, (1, 8))
    with torch.no_grad():
        got = s3m.eval()(ids, return_logits=True).logits
        want = base.eval()(ids, return_logits=True).logits
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
