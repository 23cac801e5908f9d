"""Model families on the unified decoder: Hugging Face checkpoint layout round trips and the family registry."""
import json
import os

import pytest
import torch

from paddleformers_b200.models.configuration import CONFIG_MAPPING, UNSUPPORTED_FAMILIES
from paddleformers_b200.transformers.auto import AutoConfig, AutoModelForCausalLM

TINY = dict(vocab_size=96, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=8, max_position_embeddings=64)


def _hf_names(directory):
    from safetensors import safe_open

    names = []
    for f in sorted(os.listdir(directory)):
        if f.endswith(".safetensors"):
            with safe_open(os.path.join(directory, f), "pt") as sf:
                names += list(sf.keys())
    return names


@pytest.mark.parametrize("model_type,extra,expect,absent", [
    ("llama", {}, "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.qkv_proj.weight"),
    ("mistral", {"sliding_window": 64}, "model.layers.0.mlp.gate_proj.weight", "model.layers.0.mlp.gate_up_proj.weight"),
    ("phi3", {}, "model.layers.0.self_attn.qkv_proj.weight", "model.layers.0.self_attn.q_proj.weight"),
    ("phi3", {}, "model.layers.1.mlp.gate_up_proj.weight", "model.layers.1.mlp.gate_proj.weight"),
    ("seed_oss", {}, "model.layers.0.self_attn.k_proj.bias", "model.layers.0.self_attn.qkv_proj.bias"),
    ("internlm3", {"qkv_bias": True}, "model.layers.1.self_attn.v_proj.bias", None),
    ("qwen3", {}, "model.layers.0.self_attn.q_norm.weight", None),
])
def test_family_checkpoint_roundtrip(tmp_path, model_type, extra, expect, absent):
    torch.manual_seed(0)
    cfg = AutoConfig.for_model(model_type, **{**TINY, **extra})
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    model.save_pretrained(str(tmp_path))
    names = _hf_names(str(tmp_path))
    assert expect in names and (absent is None or absent not in names)
    assert json.load(open(tmp_path / "config.json"))["model_type"] == model_type
    again = AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32)
    assert type(again) is type(model)
    ids = torch.randint(0, 96, (2, 16))
    a = model(ids, return_logits=True).logits
    b = again(ids, return_logits=True).logits
    torch.testing.assert_close(a, b, rtol=0, atol=0)


def test_mistral_sliding_window_shorter_than_sequence_is_refused():
    cfg = AutoConfig.for_model("mistral", **{**TINY, "sliding_window": 8})
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    with pytest.raises(NotImplementedError, match="sliding_window"):
        model(torch.randint(0, 96, (1, 16)), return_logits=True)


def test_registry_names_known_but_unimplemented_families():
    assert not set(CONFIG_MAPPING) & set(UNSUPPORTED_FAMILIES)
    with pytest.raises(NotImplementedError, match="attention sinks"):
        AutoConfig.for_model("gpt_oss")
    with pytest.raises(ValueError, match="unknown model_type"):
        AutoConfig.for_model("no_such_family")


def _grads(cfg_over, moe=False):
    from paddleformers_b200.models.configuration import Qwen3MoeConfig

    torch.manual_seed(3)
    if moe:
        cfg = Qwen3MoeConfig(vocab_size=96, hidden_size=32, intermediate_size=48, moe_intermediate_size=16, num_hidden_layers=2,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=8, num_experts=4, num_experts_per_tok=2,
                             router_aux_loss_coef=0.0, **cfg_over)
    else:
        cfg = AutoConfig.for_model("llama", **{**TINY, "num_hidden_layers": 4, **cfg_over})
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).train()
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, 96, (2, 16), generator=g)
    out = model(ids, labels=torch.roll(ids, -1, 1))
    out.loss.backward()
    return out.loss.item(), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


@pytest.mark.parametrize("over", [
    dict(recompute_granularity="full"),
    dict(recompute_granularity="full", recompute_method="uniform", recompute_num_layers=2),
    dict(recompute_granularity="full", recompute_method="block", recompute_num_layers=1),
    dict(recompute_granularity="selective", recompute_modules=["attn"]),
    dict(recompute_granularity="selective", recompute_modules="core_attn,mlp"),
])
def test_recompute_variants_leave_loss_and_gradients_unchanged(over):
    loss0, g0 = _grads({})
    loss1, g1 = _grads(over)
    assert loss0 == pytest.approx(loss1, rel=1e-6) and g0.keys() == g1.keys()
    for k in g0:
        torch.testing.assert_close(g0[k], g1[k], rtol=1e-5, atol=1e-7)


def test_moe_subbatching_matches_single_pass():
    loss0, g0 = _grads({}, moe=True)
    loss1, g1 = _grads({"moe_subbatch_token_num_before_dispatch": 8}, moe=True)
    assert loss0 == pytest.approx(loss1, rel=1e-5)
    for k in g0:
        torch.testing.assert_close(g0[k], g1[k], rtol=1e-4, atol=1e-6)
