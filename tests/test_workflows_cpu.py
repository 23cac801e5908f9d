"""End-to-end CPU checks of the fine-tuning workflows and of the MLA / MTP / GLM model variants."""
import os

import pytest
import torch

from paddleformers_b200 import Trainer, TrainingArguments
from paddleformers_b200.datasets.collate import dpo_collate_fn
from paddleformers_b200.models.configuration import named_config
from paddleformers_b200.transformers.auto import AutoConfig, AutoModelForCausalLM


def _tiny(**kw):
    cfg = named_config("tiny-llama", vocab_size=64, hidden_size=32, intermediate_size=64, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=16, **kw)
    torch.manual_seed(0)
    return AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)


class _Pairs(torch.utils.data.Dataset):
    """The chosen answer continues with token 7, the rejected one with token 9."""

    def __len__(self):
        return 64

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(i)
        p = torch.randint(10, 60, (6,), generator=g).tolist()
        return {"prompt_ids": p, "chosen_ids": [7, 7, 7, 1], "rejected_ids": [9, 9, 9, 1]}


@pytest.mark.parametrize("loss_type", ["sigmoid", "ipo", "simpo"])
def test_dpo_training_raises_the_reward_margin(tmp_path, loss_type):
    from paddleformers_b200.trainer.dpo_trainer import DPOTrainer

    policy, ref = _tiny(), _tiny()
    args = TrainingArguments(output_dir=str(tmp_path), per_device_train_batch_size=4, max_steps=12, learning_rate=5e-3,
                             logging_steps=1, save_strategy="no", max_seq_len=32, device="cpu", lr_scheduler_type="constant")
    tr = DPOTrainer(model=policy, ref_model=ref, args=args, train_dataset=_Pairs(), data_collator=lambda b: dpo_collate_fn(b, max_seq_len=32),
                    dpo_loss_type=loss_type, dpo_beta=0.5)
    tr.train()
    recs = [h for h in tr.state.log_history if "loss" in h]
    assert recs[-1]["loss"] < recs[0]["loss"]
    batch = dpo_collate_fn([_Pairs()[i] for i in range(8)], max_seq_len=32)
    with torch.no_grad():
        c, r, _ = tr._logps(policy, batch)
    assert (c > r).all()                                    # the policy now prefers the chosen continuation


def test_lora_finetune_trains_only_adapters_and_merges(tmp_path):
    from paddleformers_b200.data.synthetic import SyntheticCausalLMDataset
    from paddleformers_b200.peft.lora import LoRAConfig, LoRAModel

    base = _tiny()
    before = {k: v.clone() for k, v in base.state_dict().items()}
    model = LoRAModel(base, LoRAConfig(r=4, lora_alpha=8))
    args = TrainingArguments(output_dir=str(tmp_path), per_device_train_batch_size=2, max_steps=8, learning_rate=1e-2,
                             logging_steps=1, save_strategy="no", max_seq_len=16, device="cpu", lr_scheduler_type="constant")

    class Fixed(torch.utils.data.Dataset):
        ds = SyntheticCausalLMDataset(64, 16, num_samples=2, seed=0)

        def __len__(self):
            return 32

        def __getitem__(self, i):
            return self.ds[i % 2]

    tr = Trainer(model=model, args=args, train_dataset=Fixed())
    tr.train()
    losses = [h["loss"] for h in tr.state.log_history if "loss" in h]
    assert losses[-1] < losses[0]
    for k, v in base.state_dict().items():
        if "lora_" not in k and k in before:
            assert torch.equal(v, before[k]), k              # frozen base weights did not move
    ids = torch.randint(0, 64, (2, 16))
    with torch.no_grad():
        with_adapters = model(ids, return_logits=True).logits
        merged = model.merge_and_unload() if hasattr(model, "merge_and_unload") else None
    if merged is not None:
        with torch.no_grad():
            torch.testing.assert_close(merged(ids, return_logits=True).logits, with_adapters, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("preset,over", [
    ("deepseek-v3-4l", dict(hidden_size=64, intermediate_size=96, moe_intermediate_size=32, num_attention_heads=4,
                            num_key_value_heads=4, n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1,
                            q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, head_dim=24,
                            vocab_size=96, num_hidden_layers=3, first_k_dense_replace=1)),
    ("glm4.5-air-12l", dict(hidden_size=64, intermediate_size=96, moe_intermediate_size=32, num_attention_heads=4,
                            num_key_value_heads=2, head_dim=16, n_routed_experts=4, num_experts_per_tok=2, vocab_size=96,
                            num_hidden_layers=3)),
])
def test_mla_mtp_and_glm_variants_train_and_roundtrip(tmp_path, preset, over):
    torch.manual_seed(0)
    cfg = named_config(preset, **over)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    assert len(model.mtp_layers) == 1
    ids = torch.randint(0, 96, (2, 16))
    labels = torch.roll(ids, -1, 1)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    first = last = None
    for _ in range(8):
        out = model(ids, labels=labels)
        assert out.mtp_losses is not None and len(out.mtp_losses) == 1
        opt.zero_grad()
        out.loss.backward()
        opt.step()
        first = first if first is not None else out.loss.item()
        last = out.loss.item()
    assert last < first
    model.eval()
    model.save_pretrained(str(tmp_path))
    again = AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    with torch.no_grad():
        torch.testing.assert_close(model(ids, return_logits=True).logits, again(ids, return_logits=True).logits, rtol=0, atol=0)
    # the MTP block is stored as an extra entry of model.layers, like the Hugging Face checkpoints
    from safetensors import safe_open

    names = []
    for f in os.listdir(tmp_path):
        if f.endswith(".safetensors"):
            with safe_open(str(tmp_path / f), "pt") as sf:
                names += list(sf.keys())
    assert any(n.startswith(f"model.layers.{cfg.num_hidden_layers}.") and "eh_proj" in n for n in names)


def test_peft_adapter_export_and_import_preserve_the_function(tmp_path):
    """Fused-layer adapters written in the Hugging Face PEFT layout (per-projection pairs), read back into fused layers of
    a larger rank with block-diagonal B: same logits; and the per-projection tensors reproduce the delta by hand."""
    from safetensors.torch import load_file

    from paddleformers_b200.peft.hf_format import export_peft_adapter, import_peft_adapter
    from paddleformers_b200.peft.lora import LoRAConfig, LoRAModel

    base = _tiny()
    ref_state = {k: v.clone() for k, v in base.state_dict().items()}
    model = LoRAModel(base, LoRAConfig(r=4, lora_alpha=8))
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "lora_B" in n:
                p.normal_(0, 0.05)                         # B starts at zero: make the adapters matter
    ids = torch.randint(0, 64, (2, 12))
    with torch.no_grad():
        want = model(ids, return_logits=True).logits
    export_peft_adapter(model, str(tmp_path))
    sd = load_file(str(tmp_path / "adapter_model.safetensors"))
    assert "base_model.model.model.layers.0.self_attn.k_proj.lora_B.weight" in sd
    assert "base_model.model.model.layers.1.mlp.up_proj.lora_A.weight" in sd and not any("qkv_proj" in k for k in sd)
    # the per-projection pair reproduces the fused delta rows of that projection
    lin = model.model.model.layers["0"].self_attn.qkv_proj
    q_rows = base.config.num_attention_heads * base.config.head_dim
    delta_k = sd["base_model.model.model.layers.0.self_attn.k_proj.lora_B.weight"] @ sd["base_model.model.model.layers.0.self_attn.k_proj.lora_A.weight"]
    torch.testing.assert_close(delta_k * model.lora_config.scaling, lin.delta()[q_rows:q_rows + delta_k.shape[0]], rtol=1e-5, atol=1e-6)
    # a fresh copy of the base model + the PEFT directory == the adapted model
    fresh = _tiny()
    fresh.load_state_dict(ref_state)
    again = import_peft_adapter(fresh, str(tmp_path))
    assert again.lora_config.r == 12                        # q, k, v pairs stacked
    with torch.no_grad():
        torch.testing.assert_close(again(ids, return_logits=True).logits, want, rtol=1e-4, atol=1e-5)


def test_health_monitors_sample_and_truncate_on_resume(tmp_path):
    import json

    from paddleformers_b200 import AutoModelForCausalLM, Trainer, TrainingArguments
    from paddleformers_b200.data.synthetic import SyntheticCausalLMDataset
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.trainer.health_monitor import HealthMonitorCallback

    def run(steps, resume=None):
        torch.manual_seed(0)
        from paddleformers_b200.models.configuration import Qwen3MoeConfig

        cfg = Qwen3MoeConfig(vocab_size=128, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=2,
                             num_attention_heads=2, num_key_value_heads=2, head_dim=32, num_experts=4, num_experts_per_tok=2)
        model = AutoModelForCausalLM.from_config(cfg)
        args = TrainingArguments(output_dir=str(tmp_path), per_device_train_batch_size=2, max_steps=steps, learning_rate=1e-3,
                                 save_steps=4, max_seq_len=32, lr_scheduler_type="constant",
                                 internal_medicine_monitor_interval=2)
        tr = Trainer(model=model, args=args, train_dataset=SyntheticCausalLMDataset(128, 32, 64, seed=0))
        tr.train(resume_from_checkpoint=resume)
        return tr

    tr = run(6)
    cb = [c for c in tr.callback_handler.callbacks if isinstance(c, HealthMonitorCallback)][0]
    assert [r["global_step"] for r in cb.records] == [2, 4, 6]
    rec = cb.records[0]
    assert rec["act_rms/layer0"] > 0 and rec["act_absmax/layer1"] >= rec["act_rms/layer1"]
    assert rec["grad_norm/all"] > 0 and rec["weight_norm/layer0"] > 0
    assert 1.0 <= rec["router_max_share/layer0"] and 0.0 <= rec["router_entropy/layer0"] <= 1.0 + 1e-6
    assert any(k.startswith("expert_weight_norm/layer0/") for k in rec)
    path = tmp_path / "runs" / "internal_medicine.jsonl"
    assert [json.loads(l)["global_step"] for l in path.read_text().splitlines()] == [2, 4, 6]
    # resume from step 4: rows past the checkpoint are dropped, the first resumed step is not sampled
    tr2 = run(8, resume=str(tmp_path / "checkpoint-4"))
    steps = [json.loads(l)["global_step"] for l in path.read_text().splitlines()]
    assert steps == [2, 4, 6, 8] and tr2.state.global_step == 8
    # a fresh start moves the old file aside
    run(2)
    assert [json.loads(l)["global_step"] for l in path.read_text().splitlines()] == [2]
    assert any(p.name.startswith("internal_medicine.jsonl.bak.") for p in path.parent.iterdir())


def test_lora_ga_initialisation_keeps_the_function_and_follows_the_gradient():
    from paddleformers_b200 import AutoModelForCausalLM
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.peft.lora import LoRAConfig, LoRALinear, LoRAModel
    from paddleformers_b200.peft.lora_ga import estimate_gradients, lora_ga_reinit

    torch.manual_seed(0)
    cfg = named_config("tiny-llama", vocab_size=128, hidden_size=64, intermediate_size=128, num_attention_heads=2,
                       num_key_value_heads=2, head_dim=32)
    base = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    model = LoRAModel(base, LoRAConfig(r=4, lora_alpha=8))
    g = torch.Generator().manual_seed(1)
    batches = [dict(input_ids=(ids := torch.randint(0, 128, (2, 16), generator=g)), labels=torch.roll(ids, -1, 1)) for _ in range(3)]
    model.eval()
    before = model(input_ids=batches[0]["input_ids"], return_logits=True).logits.detach().clone()
    loss_before = float(model(**batches[0]).loss)
    grads = estimate_gradients(model, batches)
    layers = {n: m for n, m in model.named_modules() if isinstance(m, LoRALinear)}
    assert set(grads) == set(layers) and all(g.abs().sum() > 0 for g in grads.values())
    assert not any(m.base.weight.requires_grad or m.disabled for m in layers.values())
    lora_ga_reinit(model, grads, stable_gamma=16)
    # the function is unchanged at step 0 although the adapters are no longer zero
    after = model(input_ids=batches[0]["input_ids"], return_logits=True).logits
    assert torch.allclose(before, after, rtol=1e-4, atol=1e-4)
    name, layer = next(iter(layers.items()))
    assert layer.lora_B.abs().sum() > 0
    # B spans the top left singular directions of the gradient, A the next input-side directions
    U, S, Vh = torch.linalg.svd(grads[name], full_matrices=False)
    Bn = layer.lora_B / layer.lora_B.norm(dim=0, keepdim=True)
    assert (U[:, :4].T @ Bn).abs().diagonal().min() > 0.9
    An = layer.lora_A / layer.lora_A.norm(dim=1, keepdim=True)
    assert (An @ Vh[4:8].T).abs().diagonal().min() > 0.9
    # one SGD step on the adapters lowers the loss at least as fast as from the default initialisation
    def one_step(m, lr=0.05):
        m.train()
        loss = m(**batches[0]).loss
        loss.backward()
        with torch.no_grad():
            for p in m.parameters():
                if p.requires_grad and p.grad is not None:
                    p -= lr * p.grad
        m.eval()
        return float(m(**batches[0]).loss)

    ga = one_step(model)
    torch.manual_seed(0)
    plain = LoRAModel(AutoModelForCausalLM.from_config(cfg, dtype=torch.float32), LoRAConfig(r=4, lora_alpha=8))
    pl = one_step(plain)
    assert ga < loss_before and ga < pl


def test_lora_ga_adapters_saved_relative_to_the_original_weights(tmp_path):
    from paddleformers_b200 import AutoModelForCausalLM
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.peft.lora import LoRAConfig, LoRAModel
    from paddleformers_b200.peft.lora_ga import lora_ga_init

    torch.manual_seed(0)
    cfg = named_config("tiny-llama", vocab_size=128, hidden_size=64, intermediate_size=128, num_attention_heads=2,
                       num_key_value_heads=2, head_dim=32)
    base = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    base.save_pretrained(str(tmp_path / "base"))
    model = LoRAModel(base, LoRAConfig(r=4, lora_alpha=8))
    ids = torch.randint(0, 128, (2, 16))
    batch = dict(input_ids=ids, labels=torch.roll(ids, -1, 1))
    lora_ga_init(model, [batch])
    model.train()
    model(**batch).loss.backward()                       # one update so that B A differs from B0 A0
    with torch.no_grad():
        for p in model.parameters():
            if p.requires_grad and p.grad is not None:
                p -= 0.05 * p.grad
    model.eval()
    want = model(input_ids=ids, return_logits=True).logits.detach()
    model.save_pretrained(str(tmp_path / "adapter"))
    saved = LoRAConfig.from_pretrained(str(tmp_path / "adapter"))
    assert saved.r == 8 and saved.lora_alpha == 16 and saved.scaling == model.lora_config.scaling
    fresh = LoRAModel.from_pretrained(AutoModelForCausalLM.from_pretrained(str(tmp_path / "base"), dtype=torch.float32),
                                      str(tmp_path / "adapter")).eval()
    got = fresh(input_ids=ids, return_logits=True).logits
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-4)
    merged = fresh.merged_model()
    assert torch.allclose(merged(input_ids=ids, return_logits=True).logits, want, rtol=1e-4, atol=1e-4)
