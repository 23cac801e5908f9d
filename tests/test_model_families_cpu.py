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


def test_sliding_window_is_expressed_through_the_mask_bounds():
    """Window layers see the last ``window`` keys only; the window composes with packed-document bounds; cached decoding
    applies the same rule; context parallelism with a window is refused."""
    from paddleformers_b200.generation.utils import GenerationConfig, generate

    cfg = AutoConfig.for_model("mistral", **{**TINY, "sliding_window": 8})
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).eval()
    ids = torch.randint(0, 96, (2, 20))
    ctx = model.model.make_context(ids)
    assert ctx.kend_window.tolist()[0] == [min(j + 8, 20) for j in range(20)]
    kend = torch.full((2, 20), 20, dtype=torch.int32)
    kend[:, :5] = 5                                                      # a first document of 5 tokens
    assert model.model.make_context(ids, kend=kend).kend_window.tolist()[0][:6] == [5, 5, 5, 5, 5, 13]
    # a change more than ``window`` tokens back cannot reach a later position through ONE layer, and a sequence no longer than
    # the window is plain causal attention
    assert model.model.make_context(ids[:, :8]).kend_window is None
    with torch.no_grad():
        full = model(ids, return_logits=True).logits
        # greedy decoding with the cache agrees with a full forward under the same window rule
        out = generate(model, ids[:, :12], GenerationConfig(max_new_tokens=5))
        again = model(out[:, :-1], return_logits=True).logits
    assert torch.equal(again[:, 11:].argmax(-1), out[:, 12:])
    wide = AutoConfig.for_model("mistral", **{**TINY, "sliding_window": 64})
    torch.manual_seed(0)
    ref = AutoModelForCausalLM.from_config(wide, dtype=torch.float32).eval()
    with torch.no_grad():
        assert not torch.allclose(ref(ids, return_logits=True).logits[:, -1], full[:, -1], atol=1e-5)   # the window matters
        torch.testing.assert_close(ref(ids[:, :8], return_logits=True).logits, model(ids[:, :8], return_logits=True).logits)
    assert [cfg.layer_window(i) for i in range(2)] == [8, 8]
    q2 = AutoConfig.for_model("qwen2", **{**TINY, "sliding_window": 8, "use_sliding_window": True, "max_window_layers": 1})
    assert [q2.layer_window(i) for i in range(2)] == [0, 8]
    q3 = AutoConfig.for_model("qwen2", **{**TINY, "sliding_window": 8, "use_sliding_window": False})
    assert [q3.layer_window(i) for i in range(2)] == [0, 0]


def test_registry_names_known_but_unimplemented_families():
    assert not set(CONFIG_MAPPING) & set(UNSUPPORTED_FAMILIES)
    with pytest.raises(NotImplementedError, match="sparse"):
        AutoConfig.for_model("deepseek_v4")
    with pytest.raises(NotImplementedError, match="audio"):
        AutoConfig.for_model("qwen3_omni_moe")
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
    labels = torch.roll(ids, -1, 1)
    labels[:, :5] = -100                 # prompt positions carry no label
    labels[1, 9] = -100
    out = model(ids, labels=labels)
    out.loss.backward()
    return out.loss.item(), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


@pytest.mark.parametrize("over", [
    dict(recompute_granularity="full"),
    dict(recompute_granularity="full", recompute_method="uniform", recompute_num_layers=2),
    dict(recompute_granularity="full", recompute_method="block", recompute_num_layers=1),
    dict(recompute_granularity="selective", recompute_modules=["attn"]),
    dict(recompute_granularity="selective", recompute_modules="core_attn,mlp"),
    dict(use_filtered_label_loss=True),
    dict(loss_subbatch_sequence_length=8),
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


def _interleaved_rope(x, pos, theta):
    """Rotary embedding on adjacent pairs (2i, 2i + 1) of the last dim; x: [S, heads, D]."""
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2).float() / D))
    ang = pos[:, None].float() * inv[None]                       # [S, D/2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).flatten(-2)


def test_ernie_rope_row_permutation_preserves_attention_scores():
    """Interleaved rotation with the checkpoint's rows == half-split rotation with the permuted rows."""
    from paddleformers_b200.ops import functional as F
    from paddleformers_b200.transformers.conversion_utils import deinterleave_rope_rows, interleave_rope_rows

    torch.manual_seed(0)
    S, H, nh, D, theta = 12, 32, 2, 16, 10000.0
    x = torch.randn(S, H)
    wq, wk = torch.randn(nh * D, H), torch.randn(nh * D, H)
    pos = torch.arange(S)
    q = _interleaved_rope((x @ wq.t()).view(S, nh, D), pos, theta)
    k = _interleaved_rope((x @ wk.t()).view(S, nh, D), pos, theta)
    ref = torch.einsum("shd,thd->hst", q, k)
    wq2, wk2 = deinterleave_rope_rows(wq, D), deinterleave_rope_rows(wk, D)
    assert torch.equal(interleave_rope_rows(wq2, D), wq)
    cos, sin = F.rope_tables(S, D, theta, x.device)
    q2 = F.rope_heads((x @ wq2.t()).contiguous(), cos, sin, pos, nh, D).view(S, nh, D)
    k2 = F.rope_heads((x @ wk2.t()).contiguous(), cos, sin, pos, nh, D).view(S, nh, D)
    got = torch.einsum("shd,thd->hst", q2, k2)
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-4)


def test_ernie45_moe_config_translation_and_checkpoint_names(tmp_path):
    cfg = AutoConfig.for_model("ernie4_5_moe", vocab_size=96, hidden_size=32, intermediate_size=48, num_hidden_layers=3,
                               num_attention_heads=4, num_key_value_heads=2, head_dim=8, moe_num_experts=4, moe_k=2,
                               moe_num_shared_experts=1, moe_layer_start_index=1, moe_intermediate_size=16)
    assert (cfg.num_experts, cfg.num_experts_per_tok, cfg.n_shared_experts, cfg.first_k_dense_replace) == (4, 2, 1, 1)
    assert cfg.topk_method == "noaux_tc" and cfg.scoring_func == "softmax" and cfg.tie_word_embeddings
    assert not cfg.is_moe_layer(0) and cfg.is_moe_layer(1)
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    with torch.no_grad():
        model.model.layers["1"].mlp.gate.e_score_correction_bias.copy_(torch.tensor([0.1, -0.2, 0.3, 0.0]))
    model.save_pretrained(str(tmp_path))
    names = _hf_names(str(tmp_path))
    assert "model.layers.1.mlp.moe_statics.e_score_correction_bias" in names
    assert "model.layers.1.mlp.experts.3.down_proj.weight" in names and "model.layers.1.mlp.shared_experts.up_proj.weight" in names
    assert "model.layers.0.mlp.gate_proj.weight" in names and "lm_head.weight" not in names
    from safetensors import safe_open

    with safe_open(str(tmp_path / "model.safetensors"), "pt") as sf:
        assert tuple(sf.get_tensor("model.layers.1.mlp.moe_statics.e_score_correction_bias").shape) == (1, 4)
        q_saved = sf.get_tensor("model.layers.0.self_attn.q_proj.weight")
    # saved rows are in the interleaved order: permuting them back gives the internal q section
    from paddleformers_b200.transformers.conversion_utils import deinterleave_rope_rows

    internal_q = model.model.layers["0"].self_attn.qkv_proj.weight[:32].detach()
    torch.testing.assert_close(deinterleave_rope_rows(q_saved, 8), internal_q, rtol=0, atol=0)
    again = AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32)
    ids = torch.randint(0, 96, (2, 16))
    torch.testing.assert_close(model(ids, return_logits=True).logits, again(ids, return_logits=True).logits, rtol=0, atol=0)


def test_granite_multipliers():
    kw = {**TINY, "num_hidden_layers": 1, "tie_word_embeddings": False}
    torch.manual_seed(1)
    base = AutoModelForCausalLM.from_config(AutoConfig.for_model("granite", **kw), dtype=torch.float32).eval()
    ids = torch.randint(0, 96, (1, 12))
    ref = base(ids, return_logits=True).logits

    def variant(**mult):
        m = AutoModelForCausalLM.from_config(AutoConfig.for_model("granite", **kw, **mult), dtype=torch.float32).eval()
        m.load_state_dict(base.state_dict())
        return m

    torch.testing.assert_close(variant(logits_scaling=4.0)(ids, return_logits=True).logits, ref / 4.0, rtol=1e-5, atol=1e-6)
    # embedding multiplier == scaled embedding table
    scaled = variant()
    with torch.no_grad():
        scaled.model.embed_tokens.weight.mul_(3.0)
    torch.testing.assert_close(variant(embedding_multiplier=3.0)(ids, return_logits=True).logits,
                               scaled(ids, return_logits=True).logits, rtol=1e-5, atol=1e-6)
    # residual multiplier against the block written out by hand
    r = 0.5
    m = variant(residual_multiplier=r)
    layer = m.model.layers["0"]
    ctx = m.model.make_context(ids)
    h = m.model.embed(ids)
    h = h + r * layer.self_attn(layer.input_layernorm(h), ctx)
    h = h + r * layer.mlp(layer.post_attention_layernorm(h))
    manual = torch.nn.functional.linear(m.model.norm(h), m.lm_head.weight).view(1, 12, -1)
    torch.testing.assert_close(m(ids, return_logits=True).logits, manual, rtol=1e-4, atol=1e-5)
    # attention multiplier replaces 1 / sqrt(head_dim)
    assert variant(attention_multiplier=0.25).model.layers["0"].self_attn.scale == 0.25


def test_qwen2_moe_shared_expert_gate_and_names(tmp_path):
    cfg = AutoConfig.for_model("qwen2_moe", vocab_size=96, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                               num_attention_heads=4, num_key_value_heads=2, head_dim=8, num_experts=4, num_experts_per_tok=2,
                               moe_intermediate_size=16, shared_expert_intermediate_size=24)
    torch.manual_seed(2)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).eval()
    moe = model.model.layers["0"].mlp
    assert moe.shared_expert_gate is not None and not moe.gate.norm_topk_prob
    x = torch.randn(10, 32)
    with torch.no_grad():
        full = moe(x)
        moe.shared_expert_gate.weight.fill_(-50.0)        # sigmoid -> 0 for most tokens: only the routed experts remain
        moe.shared_expert_gate.weight[0, 0] = -50.0
        routed_only = moe(x * 0 + x.abs())                # positive inputs keep the gate's pre-activation very negative
    assert full.shape == routed_only.shape == (10, 32)
    model.save_pretrained(str(tmp_path))
    names = _hf_names(str(tmp_path))
    assert "model.layers.0.mlp.shared_expert.down_proj.weight" in names and "model.layers.0.mlp.shared_expert_gate.weight" in names
    assert "model.layers.1.mlp.shared_expert.gate_proj.weight" in names and not any("shared_experts." in n for n in names)
    again = AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    ids = torch.randint(0, 96, (2, 8))
    torch.testing.assert_close(model(ids, return_logits=True).logits, again(ids, return_logits=True).logits, rtol=0, atol=0)


def test_minicpm_scaling_maps_to_multipliers_and_kimi_uses_deepseek_blocks():
    cfg = AutoConfig.for_model("minicpm", **{**TINY, "num_hidden_layers": 4, "scale_emb": 12.0, "scale_depth": 1.4, "dim_model_base": 8})
    assert cfg.embedding_multiplier == 12.0 and cfg.residual_multiplier == pytest.approx(0.7) and cfg.logits_scaling == 4.0
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    assert model(torch.randint(0, 96, (1, 8)), return_logits=True).logits.shape == (1, 8, 96)
    k = AutoConfig.for_model("kimi_k2", num_hidden_layers=2)
    assert k.is_mla and k.topk_method == "noaux_tc"


def test_minicpm3_is_latent_attention_with_minicpm_scaling_and_half_split_rotary_rows(tmp_path):
    from safetensors.torch import load_file

    from paddleformers_b200.models.modeling import build_weight_map

    cfg = AutoConfig.for_model("minicpm3", vocab_size=96, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                               num_attention_heads=4, qk_nope_head_dim=8, qk_rope_head_dim=4, q_lora_rank=16, kv_lora_rank=8,
                               scale_emb=12.0, scale_depth=1.4, dim_model_base=8)
    assert cfg.is_mla and cfg.head_dim == 12 and cfg.v_head_dim == 8 and cfg.num_experts == 0
    assert cfg.embedding_multiplier == 12.0 and cfg.residual_multiplier == pytest.approx(1.4 / 2 ** 0.5) and cfg.logits_scaling == 4.0
    # rotate-half checkpoints: no row permutation anywhere in the weight map (DeepSeek checkpoints get one)
    assert not any(r.rope_deinterleave for r in build_weight_map(cfg).rules.values())
    ds = AutoConfig.for_model("deepseek_v2", vocab_size=96, hidden_size=32, num_hidden_layers=1, num_attention_heads=4,
                              qk_nope_head_dim=8, qk_rope_head_dim=4, q_lora_rank=16, kv_lora_rank=8, v_head_dim=8)
    assert any(r.rope_deinterleave for r in build_weight_map(ds).rules.values())
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).eval()
    ids = torch.randint(0, 96, (2, 10))
    want = model(ids, return_logits=True).logits
    model.save_pretrained(str(tmp_path))
    names = set(load_file(str(tmp_path / "model.safetensors")))
    assert {"model.layers.0.self_attn.q_a_proj.weight", "model.layers.0.self_attn.kv_a_proj_with_mqa.weight",
            "model.layers.1.self_attn.kv_b_proj.weight", "model.layers.0.mlp.gate_proj.weight"} <= names
    assert "lm_head.weight" not in names                                      # tied head
    back = AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    torch.testing.assert_close(back(ids, return_logits=True).logits, want)
    # stored rows equal the live parameter: nothing was permuted on the way out
    stored = load_file(str(tmp_path / "model.safetensors"))["model.layers.0.self_attn.q_b_proj.weight"]
    assert torch.equal(stored, model.model.layers["0"].self_attn.q_b_proj.weight.detach())


def test_attention_backends_agree_and_sinks_absorb_probability():
    from paddleformers_b200.nn.attention import AttentionInterface

    torch.manual_seed(0)
    B, S, Hq, Hkv, D = 2, 16, 4, 2, 8
    q, k, v = torch.randn(B, S, Hq, D), torch.randn(B, S, Hkv, D), torch.randn(B, S, Hkv, D)
    rows = torch.full((B, S), S, dtype=torch.int32)
    rows[0, :6] = 6                                              # two packed documents in the first row
    outs = {n: AttentionInterface.get(n)(q, k, v, rows) for n in ("flashmask", "sdpa", "eager")}
    torch.testing.assert_close(outs["sdpa"], outs["eager"], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(outs["flashmask"], outs["eager"], rtol=1e-4, atol=1e-5)
    assert set(AttentionInterface.valid_keys()) >= {"eager", "sdpa", "flashmask"}
    # sinks: a very negative sink changes nothing, a large one drains the attention output towards zero
    none = AttentionInterface.get("eager")(q, k, v, rows, sinks=torch.full((Hq,), -1e4))
    torch.testing.assert_close(none, outs["eager"], rtol=1e-5, atol=1e-6)
    drained = AttentionInterface.get("eager")(q, k, v, rows, sinks=torch.full((Hq,), 30.0))
    assert drained.abs().max() < 1e-3 * outs["eager"].abs().max() + 1e-6
    with pytest.raises(NotImplementedError):
        AttentionInterface.get("sdpa")(q, k, v, sinks=torch.zeros(Hq))


def test_layer_factories_follow_the_tensor_parallel_plan():
    import torch.nn as nn

    from paddleformers_b200.nn.layers import Embedding, Linear, LMHead, MLP, Norm

    cfg = AutoConfig.for_model("llama", **TINY)
    assert isinstance(Linear.create(8, 16, tp_plan="colwise"), nn.Linear)            # tensor-parallel degree 1: plain layers
    assert isinstance(Embedding.create(32, 8), nn.Embedding)
    assert type(Norm.create(8)).__name__ == "RMSNorm" and isinstance(Norm.create(8, norm_type="layer_norm"), nn.LayerNorm)
    mlp = MLP.create(cfg, dtype=torch.float32)
    assert mlp(torch.randn(3, cfg.hidden_size)).shape == (3, cfg.hidden_size)
    assert LMHead.create(cfg).weight.shape == (cfg.vocab_size, cfg.hidden_size)
    with pytest.raises(KeyError):
        Norm.create(8, norm_type="nope")


@pytest.mark.parametrize("policy", ["probs", "position"])
def test_router_capacity_drops_overflow_pairs(policy):
    from paddleformers_b200.models.configuration import Qwen3MoeConfig
    from paddleformers_b200.nn.moe import TopkRouter

    torch.manual_seed(0)
    cfg = Qwen3MoeConfig(hidden_size=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=8, intermediate_size=8,
                         num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, vocab_size=32, norm_topk_prob=False)
    cfg.moe_capacity_factor, cfg.moe_drop_policy = 0.5, policy
    router = TopkRouter(cfg)
    with torch.no_grad():
        router.weight.normal_(0, 1.0)
        router.weight[0] *= 4                                      # expert 0 is over-subscribed
    x = torch.randn(32, 16)
    idx, w, _ = router(x)
    cap = 8                                                        # ceil(0.5 * 32 * 2 / 4)
    kept = w > 0
    for e in range(4):
        on_e = idx == e
        assert int((kept & on_e).sum()) == min(cap, int(on_e.sum()))
    assert int((idx == 0).sum()) > cap                             # something was actually dropped
    if policy == "position":
        pairs = torch.nonzero(idx == 0)                            # row-major: earliest tokens first
        assert kept[idx == 0][:cap].all() and not kept[idx == 0][cap:].any() and len(pairs) > cap
    else:
        router.capacity_factor = 0.0                               # same router without the cap: the original weights
        _, w_full, _ = router(x)
        on0 = idx == 0
        assert w_full[on0 & kept].min() >= w_full[on0 & ~kept].max()       # the most probable pairs survive


def test_attention_implementation_switch_matches_default_path():
    cfg = AutoConfig.for_model("llama", **TINY)
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).eval()
    ids = torch.randint(0, 96, (2, 12))
    ref = model(ids, return_logits=True).logits
    for impl in ("eager", "sdpa"):
        model.config._attn_implementation = impl
        torch.testing.assert_close(model(ids, return_logits=True).logits, ref, rtol=1e-4, atol=1e-5)


def test_sequence_level_balance_loss_is_the_mean_of_per_sequence_losses():
    from paddleformers_b200.models.configuration import Qwen3MoeConfig
    from paddleformers_b200.nn.moe import TopkRouter

    torch.manual_seed(0)
    cfg = Qwen3MoeConfig(hidden_size=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=8, intermediate_size=8,
                         num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=2, vocab_size=32,
                         router_aux_loss_coef=0.01)
    router = TopkRouter(cfg).train()
    with torch.no_grad():
        router.weight.normal_(0, 1.0)
    x = torch.randn(3 * 8, 16)
    per_seq = torch.stack([router(x[i * 8:(i + 1) * 8])[2] for i in range(3)]).mean()
    batch = router(x)[2]
    router.balance_type, router.tokens_per_seq = "seq_aux_loss", 8
    seq = router(x)[2]
    assert torch.allclose(seq, per_seq, rtol=1e-5, atol=1e-8)
    assert not torch.allclose(seq, batch, rtol=1e-4, atol=0)
    router.tokens_per_seq = 0                               # unknown layout: falls back to the batch-level term
    assert torch.allclose(router(x)[2], batch)
    router.balance_type = "none"
    assert float(router(x)[2]) == 0.0
    # end to end: the model sets the rows per sequence and the loss back-propagates into the router
    mcfg = AutoConfig.for_model("qwen3_moe", **dict(TINY, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                                                    router_aux_loss_coef=0.01, moe_router_load_balancing_type="seq_aux_loss"))
    model = AutoModelForCausalLM.from_config(mcfg, dtype=torch.float32).train()
    ids = torch.randint(0, 96, (2, 12))
    out = model(ids, labels=ids)
    (out[0] if isinstance(out, tuple) else out.loss).backward()
    gate = model.model.layers["0"].mlp.gate
    assert gate.tokens_per_seq == 12 and gate.weight.grad.abs().sum() > 0


def test_gpt_oss_trains_sinks_router_bias_and_expert_biases():
    from paddleformers_b200.generation.utils import GenerationConfig, generate

    cfg = AutoConfig.for_model("gpt_oss", **{**TINY, "num_hidden_layers": 2, "num_local_experts": 4, "num_experts_per_tok": 2,
                                            "intermediate_size": 24, "sliding_window": 6, "router_aux_loss_coef": 0.01})
    assert [cfg.layer_window(i) for i in range(2)] == [6, 0] and cfg.scoring_func == "softmax_topk"
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).train()
    ids = torch.randint(0, 96, (2, 14))
    out = model(ids, labels=torch.roll(ids, -1, 1))
    out.loss.backward()
    layer = model.model.layers["0"]
    for p in (layer.self_attn.sinks, layer.mlp.gate.bias, layer.mlp.experts.gate_up_bias, layer.mlp.experts.down_bias,
              layer.mlp.experts.gate_up_proj, layer.self_attn.o_proj.bias):
        assert p.grad is not None and p.grad.abs().sum() > 0
    assert out.aux_loss is not None
    model.eval()
    with torch.no_grad():
        seq = generate(model, ids[:, :8], GenerationConfig(max_new_tokens=4))
        again = model(seq[:, :-1], return_logits=True).logits
    assert torch.equal(again[:, 7:].argmax(-1), seq[:, 8:])          # cached decoding applies sinks and windows too


def test_llama4_chunked_layers_and_cached_decoding():
    from paddleformers_b200.generation.utils import GenerationConfig, generate

    cfg = AutoConfig.for_model("llama4_text", **{**TINY, "intermediate_size": 24, "intermediate_size_mlp": 48, "num_hidden_layers": 4,
                                                 "num_local_experts": 4, "attention_chunk_size": 6, "interleave_moe_layer_step": 2,
                                                 "floor_scale": 4})
    assert cfg.no_rope_layers == [1, 1, 1, 0] and [cfg.layer_chunk(i) for i in range(4)] == [6, 6, 6, 0] and cfg.moe_layers == [1, 3]
    assert [cfg.is_moe_layer(i) for i in range(4)] == [False, True, False, True]
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    ids = torch.randint(0, 96, (2, 15))
    ctx = model.model.make_context(ids)
    assert ctx.kend_window.tolist()[0] == [6] * 6 + [12] * 6 + [15] * 3
    out = model.train()(ids, labels=torch.roll(ids, -1, 1))
    out.loss.backward()
    moe = model.model.layers["1"].mlp
    assert moe.gate.weight.grad.abs().sum() > 0 and moe.experts.gate_up_proj.grad.abs().sum() > 0     # weights on the expert input
    model.eval()
    with torch.no_grad():
        seq = generate(model, ids[:, :9], GenerationConfig(max_new_tokens=5))
        again = model(seq[:, :-1], return_logits=True).logits
    assert torch.equal(again[:, 8:].argmax(-1), seq[:, 9:])


def test_gated_delta_rule_chunked_form_and_qwen3_next_training_step():
    from paddleformers_b200.generation.utils import GenerationConfig, generate
    from paddleformers_b200.nn.linear_attention import gated_delta_rule, gated_delta_rule_reference

    torch.manual_seed(0)
    B, S, H, dk, dv = 2, 37, 3, 8, 6
    q = torch.nn.functional.normalize(torch.randn(B, S, H, dk), dim=-1).requires_grad_(True)
    k = torch.nn.functional.normalize(torch.randn(B, S, H, dk), dim=-1).requires_grad_(True)
    v = torch.randn(B, S, H, dv, requires_grad=True)
    g, beta = -torch.rand(B, S, H) * 0.5, torch.rand(B, S, H)
    ref, s_ref = gated_delta_rule_reference(q, k, v, g, beta)
    grads_ref = torch.autograd.grad(ref.square().sum(), (q, k, v))
    for chunk in (4, 16, 64):                                    # ragged last chunk, one chunk, several chunks
        out, s_out = gated_delta_rule(q, k, v, g, beta, chunk=chunk)
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(s_out, s_ref, rtol=1e-4, atol=1e-5)
        for a, b in zip(torch.autograd.grad(out.square().sum(), (q, k, v)), grads_ref):
            torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-4)
    # the state carries over: two halves with the state passed on equal one pass
    o1, st = gated_delta_rule(q[:, :20], k[:, :20], v[:, :20], g[:, :20], beta[:, :20], chunk=8)
    o2, _ = gated_delta_rule(q[:, 20:], k[:, 20:], v[:, 20:], g[:, 20:], beta[:, 20:], chunk=8, state=st)
    torch.testing.assert_close(torch.cat([o1, o2], 1), ref, rtol=1e-4, atol=1e-5)

    cfg = AutoConfig.for_model("qwen3_next", **{**TINY, "num_hidden_layers": 4, "linear_num_value_heads": 4, "linear_num_key_heads": 2,
                                               "linear_key_head_dim": 8, "linear_value_head_dim": 8, "num_experts": 4,
                                               "num_experts_per_tok": 2, "moe_intermediate_size": 16,
                                               "shared_expert_intermediate_size": 24})
    assert cfg.layer_types == ["linear_attention"] * 3 + ["full_attention"]
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).train()
    ids = torch.randint(0, 96, (2, 13))
    out = model(ids, labels=torch.roll(ids, -1, 1))
    out.loss.backward()
    lin, full = model.model.layers["0"].linear_attn, model.model.layers["3"].self_attn
    for p in (lin.A_log, lin.dt_bias, lin.conv1d.weight, lin.in_proj_ba.weight, lin.norm.weight, full.q_proj.weight,
              model.model.layers["0"].mlp.shared_expert_gate.weight):
        assert p.grad is not None and p.grad.abs().sum() > 0
    model.eval()
    with torch.no_grad():
        seq = generate(model, ids[:, :7], GenerationConfig(max_new_tokens=3))
        again = model(seq[:, :-1], return_logits=True).logits
    assert torch.equal(again[:, 6:].argmax(-1), seq[:, 7:])


def test_sparse_indexer_attention_selects_keys_only_beyond_its_budget():
    kw = dict(vocab_size=96, hidden_size=32, intermediate_size=48, moe_intermediate_size=16, num_hidden_layers=2, num_attention_heads=2,
              n_routed_experts=4, num_experts_per_tok=2, n_group=1, topk_group=1, first_k_dense_replace=1, q_lora_rank=16, kv_lora_rank=8,
              qk_nope_head_dim=8, qk_rope_head_dim=4, v_head_dim=8, num_nextn_predict_layers=0, index_n_heads=2, index_head_dim=8)
    torch.manual_seed(0)
    sparse = AutoModelForCausalLM.from_config(AutoConfig.for_model("deepseek_v32", index_topk=6, **kw), dtype=torch.float32)
    dense_cfg = AutoConfig.for_model("deepseek_v32", index_topk=64, **kw)
    dense = AutoModelForCausalLM.from_config(dense_cfg, dtype=torch.float32)
    dense.load_state_dict(sparse.state_dict())
    ids = torch.randint(0, 96, (2, 14))
    with torch.no_grad():
        a = sparse.eval()(ids, return_logits=True).logits
        b = dense.eval()(ids, return_logits=True).logits
    # the first 6 positions have at most 6 visible keys: nothing to drop; later positions lose keys
    torch.testing.assert_close(a[:, :6], b[:, :6], rtol=1e-4, atol=1e-5)
    assert not torch.allclose(a[:, 8:], b[:, 8:], atol=1e-4)
    att = sparse.model.layers["0"].self_attn
    ctx = sparse.model.make_context(ids)
    x = sparse.model.embed(ids)
    qa = att.q_a_layernorm(att.q_a_proj(x))
    allowed = torch.ones(14, 14, dtype=torch.bool).tril()[None].expand(2, 14, 14)
    vis = att.indexer.visible(x, qa, ctx, allowed)
    assert (vis.sum(-1) == torch.arange(1, 15).clamp(max=6)[None]).all() and not (vis & ~allowed).any()
    out = sparse.train()(ids, labels=torch.roll(ids, -1, 1))
    out.loss.backward()
    assert att.kv_b_proj.weight.grad.abs().sum() > 0 and att.indexer.wk.weight.grad is None      # selection is not differentiated


def test_decayed_linear_attention_matches_the_double_sum():
    from paddleformers_b200.nn.linear_attention import decayed_linear_attention

    torch.manual_seed(0)
    B, S, H, D = 2, 21, 3, 4
    q, k, v = (torch.randn(B, S, H, D) for _ in range(3))
    slope = torch.tensor([0.5, 0.1, 0.02])
    ref = torch.zeros(B, S, H, D)
    for t in range(S):
        for i in range(t + 1):
            ref[:, t] += torch.exp(-slope * (t - i))[None, :, None] * (q[:, t] * k[:, i]).sum(-1, keepdim=True) * v[:, i]
    for chunk in (4, 8, 64):
        out, state = decayed_linear_attention(q, k, v, slope, chunk)
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    first, st = decayed_linear_attention(q[:, :9], k[:, :9], v[:, :9], slope, 4)
    rest, _ = decayed_linear_attention(q[:, 9:], k[:, 9:], v[:, 9:], slope, 4, state=st)
    torch.testing.assert_close(torch.cat([first, rest], 1), ref, rtol=1e-4, atol=1e-5)


def test_linear_attention_layers_decode_incrementally():
    """Generation keeps the convolution tail and the recurrent state of linear-attention layers (and the keys / values of the
    softmax layers): the tokens equal those of a full forward over the generated prefix, for both mixer kinds."""
    from paddleformers_b200.generation.utils import GenerationConfig, KVCache, generate

    mm = AutoConfig.for_model("minimax", **{**TINY, "num_hidden_layers": 4, "num_local_experts": 4, "num_experts_per_tok": 2,
                                            "intermediate_size": 24, "block_size": 4})
    nx = AutoConfig.for_model("qwen3_next", **{**TINY, "num_hidden_layers": 4, "linear_num_value_heads": 4, "linear_num_key_heads": 2,
                                              "linear_key_head_dim": 8, "linear_value_head_dim": 8})
    for cfg in (mm, nx):
        torch.manual_seed(0)
        model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32).eval()
        ids = torch.randint(0, 96, (2, 9))
        with torch.no_grad():
            seq = generate(model, ids, GenerationConfig(max_new_tokens=6))
            full = model(seq[:, :-1], return_logits=True).logits
            assert torch.equal(full[:, 8:].argmax(-1), seq[:, 9:])
            # the cached path itself: prefix, then one token at a time, against the full forward
            caches = {i: KVCache() for i in model.model.layer_range}
            a = model(seq[:, :9], position_ids=torch.arange(9)[None].expand(2, -1), caches=caches, return_logits=True).logits
            b = model(seq[:, 9:10], position_ids=torch.full((2, 1), 9), caches=caches, return_logits=True).logits
            torch.testing.assert_close(torch.cat([a, b], 1), model(seq[:, :10], return_logits=True).logits, rtol=1e-4, atol=1e-4)


def test_minicpm4_1_and_paligemma2_registrations(tmp_path):
    """Families that reuse an implemented architecture under their own ``model_type``: MiniCPM 4.1 (MiniCPM scaling + long-rope
    factors; the sparse-prefill description is carried in the configuration, attention stays dense) and PaliGemma 2 (the PaliGemma
    composite with a Gemma 2 decoder by default)."""
    from paddleformers_b200.transformers.auto import AutoModelForCausalLM, AutoModelForConditionalGeneration

    short, long = [1.0 + 0.05 * i for i in range(8)], [1.5 + 0.2 * i for i in range(8)]
    cfg = AutoConfig.for_model(
        "minicpm4_1", vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, scale_emb=12, scale_depth=1.4, dim_model_base=32, max_position_embeddings=64,
        rope_scaling={"rope_type": "longrope", "short_factor": short, "long_factor": long, "original_max_position_embeddings": 32},
        sparse_config={"kernel_size": 32, "kernel_stride": 16, "block_size": 64, "topk": 64, "dense_len": 8192})
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    ids = torch.randint(0, 200, (2, 16))
    model(ids, labels=ids).loss.backward()
    model.save_pretrained(str(tmp_path / "m"))
    again = AutoModelForCausalLM.from_pretrained(str(tmp_path / "m"), dtype=torch.float32)
    assert type(again).__name__ == "MiniCPM4_1ForCausalLM" and again.config.sparse_config["dense_len"] == 8192
    assert torch.equal(again(ids).logits, model(ids).logits)

    from paddleformers_b200.models.paligemma import PaliGemma2Config

    pg = PaliGemma2Config(
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, image_size=16, patch_size=8),
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                         head_dim=16, vocab_size=300, sliding_window=4, query_pre_attn_scalar=16),
        image_token_index=299, projection_dim=64)
    assert pg.text_config.model_type == "gemma2" and pg.num_image_tokens == 4
    vl = AutoModelForConditionalGeneration.from_config(pg, dtype=torch.float32)
    vl.save_pretrained(str(tmp_path / "pg"))
    back = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "pg"), dtype=torch.float32)
    ids = torch.tensor([[299] * 4 + [2, 5, 6, 7, 8, 9]])
    pixels = torch.randn(1, 3, 16, 16)
    types = torch.tensor([[0] * 6 + [1] * 4])
    assert back.config.model_type == "paligemma2"
    assert torch.equal(back(ids, pixel_values=pixels, token_type_ids=types).logits, vl(ids, pixel_values=pixels, token_type_ids=types).logits)
