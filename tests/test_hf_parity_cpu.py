"""Parity with the Hugging Face ``transformers`` PyTorch implementations, used as an independent oracle: a tiny randomly
initialised HF model is saved as safetensors, loaded through this framework's weight maps, and must produce the same
logits (fp32, CPU). This pins the rotary conventions, fused-projection layouts, router rules, MLA and the per-family
multipliers to an implementation that shares no code with this repository."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from paddleformers_b200.transformers.auto import AutoModelForCausalLM  # noqa: E402

BASE = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=128, tie_word_embeddings=False)

CASES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", dict(rope_theta=10000.0, rms_norm_eps=1e-5)),
    "llama_theta": ("LlamaConfig", "LlamaForCausalLM", dict(rope_theta=500000.0)),
    "llama3_scaling": ("LlamaConfig", "LlamaForCausalLM", dict(rope_theta=500000.0, rope_scaling={
        "rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 16})),
    "llama_linear_scaling": ("LlamaConfig", "LlamaForCausalLM", dict(rope_scaling={"rope_type": "linear", "factor": 4.0})),
    "llama_biases_tied": ("LlamaConfig", "LlamaForCausalLM", dict(attention_bias=True, mlp_bias=True, tie_word_embeddings=True, head_dim=32)),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(sliding_window=None)),
    "mistral_sliding_window": ("MistralConfig", "MistralForCausalLM", dict(sliding_window=8)),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", dict()),
    "qwen2_sliding_upper_layers": ("Qwen2Config", "Qwen2ForCausalLM", dict(num_hidden_layers=3, use_sliding_window=True, sliding_window=6,
                                                                          max_window_layers=1)),
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(head_dim=16)),
    "phi3": ("Phi3Config", "Phi3ForCausalLM", dict(pad_token_id=0)),
    "phi3_longrope": ("Phi3Config", "Phi3ForCausalLM", dict(pad_token_id=0, original_max_position_embeddings=16, rope_scaling={
        "rope_type": "longrope", "short_factor": [1.0, 1.1, 1.2, 1.3, 1.4, 1.5, 1.6, 1.7],
        "long_factor": [1.5, 2.0, 2.5, 3.0, 3.5, 4.0, 4.5, 5.0]})),
    "llama_dynamic_ntk": ("LlamaConfig", "LlamaForCausalLM", dict(max_position_embeddings=16, rope_scaling={"rope_type": "dynamic", "factor": 2.0})),
    "seed_oss": ("SeedOssConfig", "SeedOssForCausalLM", dict(head_dim=16)),
    "granite": ("GraniteConfig", "GraniteForCausalLM", dict(embedding_multiplier=3.0, residual_multiplier=0.5, attention_multiplier=0.2,
                                                           logits_scaling=2.0)),
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", dict(head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                                                               norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[])),
    "qwen3_moe_mixed_layers": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", dict(
        head_dim=16, num_hidden_layers=4, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, norm_topk_prob=False,
        decoder_sparse_step=2, mlp_only_layers=[1])),
    "deepseek_v3_groups": ("DeepseekV3Config", "DeepseekV3ForCausalLM", dict(
        num_hidden_layers=3, num_key_value_heads=4, moe_intermediate_size=32, n_routed_experts=16, num_experts_per_tok=4, n_group=4,
        topk_group=2, n_shared_experts=2, first_k_dense_replace=2, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16,
        qk_rope_head_dim=8, v_head_dim=16, routed_scaling_factor=1.0, norm_topk_prob=False)),
    "glm4_moe_plain": ("Glm4MoeConfig", "Glm4MoeForCausalLM", dict(
        head_dim=16, moe_intermediate_size=32, n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1, n_shared_experts=1,
        first_k_dense_replace=0, partial_rotary_factor=0.5, use_qk_norm=False, attention_bias=True, routed_scaling_factor=1.0,
        norm_topk_prob=True)),
    "qwen2_moe": ("Qwen2MoeConfig", "Qwen2MoeForCausalLM", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                                                               shared_expert_intermediate_size=48, norm_topk_prob=False,
                                                               decoder_sparse_step=1, mlp_only_layers=[])),
    "ernie4_5": ("Ernie4_5Config", "Ernie4_5ForCausalLM", dict(head_dim=16, tie_word_embeddings=True)),
    "ernie4_5_moe": ("Ernie4_5_MoeConfig", "Ernie4_5_MoeForCausalLM", dict(head_dim=16, tie_word_embeddings=True, moe_num_experts=4, moe_k=2,
                                                                         moe_intermediate_size=32, moe_num_shared_experts=1,
                                                                         moe_layer_start_index=1, moe_layer_interval=1)),
    "deepseek_v3": ("DeepseekV3Config", "DeepseekV3ForCausalLM", dict(num_key_value_heads=4, moe_intermediate_size=32, n_routed_experts=8,
                                                                     num_experts_per_tok=2, n_group=2, topk_group=1, n_shared_experts=1,
                                                                     first_k_dense_replace=1, q_lora_rank=24, kv_lora_rank=16,
                                                                     qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                                                                     routed_scaling_factor=2.5, norm_topk_prob=True)),
    "deepseek_v3_yarn": ("DeepseekV3Config", "DeepseekV3ForCausalLM", dict(
        num_key_value_heads=4, moe_intermediate_size=32, n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1,
        n_shared_experts=1, first_k_dense_replace=1, q_lora_rank=None, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
        v_head_dim=16, routed_scaling_factor=2.5, norm_topk_prob=True, max_position_embeddings=128,
        rope_scaling={"rope_type": "yarn", "factor": 4.0, "beta_fast": 32, "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 0.707,
                      "original_max_position_embeddings": 32})),
    "deepseek_v2": ("DeepseekV2Config", "DeepseekV2ForCausalLM", dict(
        num_key_value_heads=4, moe_intermediate_size=32, n_routed_experts=8, num_experts_per_tok=2, n_group=2, topk_group=1,
        n_shared_experts=1, first_k_dense_replace=1, q_lora_rank=None, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
        v_head_dim=16, routed_scaling_factor=1.0, topk_method="greedy", norm_topk_prob=False)),
    "olmo2": ("Olmo2Config", "Olmo2ForCausalLM", dict()),
    "gemma": ("GemmaConfig", "GemmaForCausalLM", dict(head_dim=16, tie_word_embeddings=True, hidden_activation="gelu_pytorch_tanh")),
    "gemma2": ("Gemma2Config", "Gemma2ForCausalLM", dict(head_dim=16, num_hidden_layers=4, sliding_window=8, query_pre_attn_scalar=24,
                                                        attn_logit_softcapping=5.0, final_logit_softcapping=3.0, tie_word_embeddings=True)),
    "gemma3_text": ("Gemma3TextConfig", "Gemma3ForCausalLM", dict(head_dim=16, num_hidden_layers=4, sliding_window=8, query_pre_attn_scalar=24,
                                                                  layer_types=["sliding_attention", "sliding_attention", "full_attention",
                                                                               "sliding_attention"], tie_word_embeddings=True)),
    "cohere": ("CohereConfig", "CohereForCausalLM", dict(tie_word_embeddings=True, logit_scale=0.25, use_qk_norm=False)),
    "cohere2": ("Cohere2Config", "Cohere2ForCausalLM", dict(tie_word_embeddings=True, logit_scale=0.25, num_hidden_layers=4, sliding_window=8,
                                                          layer_types=["sliding_attention", "full_attention", "sliding_attention",
                                                                       "full_attention"])),
    "hunyuan_v1_dense": ("HunYuanDenseV1Config", "HunYuanDenseV1ForCausalLM", dict(head_dim=16, rope_parameters={
        "rope_type": "dynamic", "alpha": 50.0, "factor": 1.0, "rope_theta": 10000.0})),
    "hunyuan_v1_moe": ("HunYuanMoEV1Config", "HunYuanMoEV1ForCausalLM", dict(head_dim=16, num_experts=4, moe_topk=2)),
    "minimax_m2": ("MiniMaxM2Config", "MiniMaxM2ForCausalLM", dict(head_dim=16, num_local_experts=4, num_experts_per_tok=2)),
    "gpt_oss": ("GptOssConfig", "GptOssForCausalLM", dict(
        head_dim=16, intermediate_size=48, num_hidden_layers=4, num_local_experts=4, num_experts_per_tok=2, sliding_window=8,
        rope_parameters={"rope_type": "yarn", "factor": 4.0, "beta_fast": 32.0, "beta_slow": 1.0, "truncate": False,
                         "original_max_position_embeddings": 32, "rope_theta": 10000.0})),
    "llama4_text": ("Llama4TextConfig", "Llama4ForCausalLM", dict(
        head_dim=16, intermediate_size=48, intermediate_size_mlp=96, num_hidden_layers=4, num_local_experts=4, num_experts_per_tok=1,
        attention_chunk_size=8, interleave_moe_layer_step=2, floor_scale=4, attn_scale=0.3)),
    "llama4_text_top2_all_moe": ("Llama4TextConfig", "Llama4ForCausalLM", dict(
        head_dim=16, intermediate_size=48, intermediate_size_mlp=96, num_hidden_layers=4, num_local_experts=4, num_experts_per_tok=2,
        attention_chunk_size=16, interleave_moe_layer_step=1, use_qk_norm=False, attn_temperature_tuning=False)),
    "qwen3_next": ("Qwen3NextConfig", "Qwen3NextForCausalLM", dict(
        head_dim=16, num_hidden_layers=4, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=8, linear_value_head_dim=8,
        num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=48, decoder_sparse_step=1,
        mlp_only_layers=[1])),
    "qwen3_5_text": ("Qwen3_5TextConfig", "Qwen3_5ForCausalLM", dict(
        head_dim=16, num_hidden_layers=4, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=8, linear_value_head_dim=8)),
    "qwen3_5_moe_text": ("Qwen3_5MoeTextConfig", "Qwen3_5MoeForCausalLM", dict(
        head_dim=16, num_hidden_layers=4, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=8, linear_value_head_dim=8,
        num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=48)),
    "glm4_moe_lite": ("Glm4MoeLiteConfig", "Glm4MoeLiteForCausalLM", dict(
        num_hidden_layers=3, num_key_value_heads=4, moe_intermediate_size=32, n_routed_experts=8, num_experts_per_tok=2, n_group=1,
        topk_group=1, n_shared_experts=1, mlp_layer_types=["dense", "sparse", "sparse"], q_lora_rank=24, kv_lora_rank=16,
        qk_nope_head_dim=24, qk_rope_head_dim=8, v_head_dim=32, routed_scaling_factor=1.8, norm_topk_prob=True)),
    "glm_moe_dsa": ("GlmMoeDsaConfig", "GlmMoeDsaForCausalLM", dict(
        num_hidden_layers=2, num_key_value_heads=4, moe_intermediate_size=32, n_routed_experts=4, num_experts_per_tok=2, n_group=1,
        topk_group=1, mlp_layer_types=["dense", "sparse"], q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8,
        v_head_dim=16, index_topk=8, index_n_heads=2, index_head_dim=16)),
    "minimax": ("MiniMaxConfig", "MiniMaxForCausalLM", dict(
        head_dim=16, intermediate_size=48, num_hidden_layers=4, num_local_experts=4, num_experts_per_tok=2, block_size=8,
        full_attn_alpha_factor=1.5, full_attn_beta_factor=0.8, linear_attn_alpha_factor=1.2, linear_attn_beta_factor=0.9,
        mlp_alpha_factor=1.1, mlp_beta_factor=0.7)),
    "diffllama": ("DiffLlamaConfig", "DiffLlamaForCausalLM", dict(num_hidden_layers=3)),
    "mixtral": ("MixtralConfig", "MixtralForCausalLM", dict(num_local_experts=4, num_experts_per_tok=2, sliding_window=8)),
    "stablelm": ("StableLmConfig", "StableLmForCausalLM", dict(use_qkv_bias=True, partial_rotary_factor=0.25)),
    "glm4_moe": ("Glm4MoeConfig", "Glm4MoeForCausalLM", dict(head_dim=16, moe_intermediate_size=32, n_routed_experts=4, num_experts_per_tok=2,
                                                             n_group=1, topk_group=1, n_shared_experts=1, first_k_dense_replace=1,
                                                             partial_rotary_factor=0.5, use_qk_norm=True, routed_scaling_factor=1.5,
                                                             norm_topk_prob=True)),
}


@pytest.mark.parametrize("family", sorted(CASES))
def test_logits_match_hugging_face_implementation(tmp_path, family):
    cfg_name, cls_name, extra = CASES[family]
    if not (hasattr(transformers, cfg_name) and hasattr(transformers, cls_name)):
        pytest.skip(f"transformers has no {cls_name}")
    torch.manual_seed(0)
    hf_cfg = getattr(transformers, cfg_name)(**{**BASE, **extra})
    if family == "glm_moe_dsa":
        hf_cfg._attn_implementation = "eager"      # its default attention path drops the causal mask when no mask tensor is passed
    hf = getattr(transformers, cls_name)(hf_cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():          # non-trivial values everywhere (norm weights, router biases)
            if p.dim() == 1 or n.endswith("bias"):
                p.normal_(1.0 if "norm" in n else 0.0, 0.1)
        for n, b in hf.named_buffers():
            if "e_score_correction_bias" in n:
                b.normal_(0.0, 0.1)
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    mine = AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    ids = torch.randint(0, 128, (2, 24))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = mine(ids, return_logits=True).logits
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("family", ["llama", "qwen3", "qwen3_moe", "deepseek_v3", "glm4_moe", "ernie4_5", "phi3", "gemma", "gemma2", "gemma3_text", "cohere", "cohere2", "olmo2", "hunyuan_v1_dense", "hunyuan_v1_moe", "minimax_m2", "mixtral", "deepseek_v2", "gpt_oss", "llama4_text", "qwen3_next", "qwen3_5_text", "qwen3_5_moe_text", "glm4_moe_lite", "glm_moe_dsa", "minimax", "diffllama",
                                    "stablelm", "granite", "qwen2_moe", "ernie4_5_moe"])
def test_hugging_face_loads_what_this_framework_saves(tmp_path, family):
    """The other direction: a checkpoint written by ``save_pretrained`` here (per-expert tensors, interleaved rotary rows
    restored, HF config field names) loads in ``transformers`` and gives the same logits."""
    cfg_name, cls_name, extra = CASES[family]
    torch.manual_seed(1)
    hf_cfg = getattr(transformers, cfg_name)(**{**BASE, **extra})
    src = tmp_path / "src"
    getattr(transformers, cls_name)(hf_cfg).save_pretrained(str(src), safe_serialization=True)
    mine = AutoModelForCausalLM.from_pretrained(str(src), dtype=torch.float32).eval()
    out = tmp_path / "out"
    mine.save_pretrained(str(out))
    back = getattr(transformers, cls_name).from_pretrained(str(out), torch_dtype=torch.float32,
                                                           **({"attn_implementation": "eager"} if family == "glm_moe_dsa" else {})).eval()
    ids = torch.randint(0, 128, (2, 24))
    with torch.no_grad():
        torch.testing.assert_close(back(input_ids=ids).logits, mine(ids, return_logits=True).logits, rtol=2e-4, atol=2e-4)


def test_loss_gradients_and_greedy_generation_match_hugging_face(tmp_path):
    """Loss convention (targets shifted by the data pipeline here, inside the model there), gradients of the fused qkv /
    gate|up parameters against the concatenated Hugging Face gradients, and cached greedy decoding."""
    from paddleformers_b200.generation.utils import GenerationConfig, generate

    torch.manual_seed(3)
    hf_cfg = transformers.LlamaConfig(**{**BASE, "rope_theta": 10000.0})
    hf = transformers.LlamaForCausalLM(hf_cfg).float()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    mine = AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32)
    ids = torch.randint(1, 128, (2, 20))        # 0 is the pad id below: transformers masks pad tokens found in a prompt
    labels = torch.cat([ids[:, 1:], torch.full((2, 1), -100)], dim=1)          # next-token targets, last position ignored
    out = mine(ids, labels=labels)
    want = hf(input_ids=ids, labels=ids)
    assert out.loss.item() == pytest.approx(want.loss.item(), rel=1e-5)
    out.loss.backward()
    want.loss.backward()
    layer, hl = mine.model.layers["0"], hf.model.layers[0]
    g_qkv = torch.cat([hl.self_attn.q_proj.weight.grad, hl.self_attn.k_proj.weight.grad, hl.self_attn.v_proj.weight.grad])
    torch.testing.assert_close(layer.self_attn.qkv_proj.weight.grad, g_qkv, rtol=1e-4, atol=1e-6)
    g_gu = torch.cat([hl.mlp.gate_proj.weight.grad, hl.mlp.up_proj.weight.grad])
    torch.testing.assert_close(layer.mlp.gate_up_proj.weight.grad, g_gu, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(mine.model.embed_tokens.weight.grad, hf.model.embed_tokens.weight.grad, rtol=1e-4, atol=1e-6)
    prompt = ids[:, :6]
    mine.eval(); hf.eval()
    got = generate(mine, prompt, GenerationConfig(max_new_tokens=8))
    ref = hf.generate(prompt, max_new_tokens=8, do_sample=False, pad_token_id=0)
    assert torch.equal(got, ref)


def test_qwen2_vl_matches_hugging_face(tmp_path):
    """Vision tower (2-D rotary, merge-block patch order, patch merger), placeholder scatter and multimodal rotary
    positions against ``transformers``' Qwen2-VL on two images of different sizes between text tokens."""
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(5)
    vc = dict(depth=2, embed_dim=32, hidden_size=64, mlp_ratio=2, num_heads=2, in_channels=3, patch_size=4, spatial_merge_size=2,
              temporal_patch_size=2)
    tc = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              max_position_embeddings=128, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, tie_word_embeddings=False)
    cfg = transformers.Qwen2VLConfig(text_config=tc, vision_config=vc, image_token_id=120, video_token_id=121,
                                     vision_start_token_id=118, vision_end_token_id=119)
    hf = transformers.Qwen2VLForConditionalGeneration(cfg).eval().float()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    grid = torch.tensor([[1, 4, 6], [1, 2, 2]])                       # patches before merging: 24 and 4 -> 6 and 1 tokens
    pixels = torch.randn(int(grid.prod(-1).sum()), 3 * 2 * 4 * 4)
    ids = torch.tensor([[5, 6, 118] + [120] * 6 + [119, 7, 8, 9, 118, 120, 119, 10, 11]])
    types = (ids == 120).int()
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits
        got = mine(ids, pixel_values=pixels, image_grid_thw=grid, return_logits=True).logits
    torch.testing.assert_close(got, want, rtol=3e-4, atol=3e-4)
    # text only: identical to the plain decoder path
    text = torch.randint(0, 100, (2, 12))
    with torch.no_grad():
        torch.testing.assert_close(mine(text, return_logits=True).logits, hf(input_ids=text).logits, rtol=3e-4, atol=3e-4)
    # round trip through this framework's writer, read back by transformers
    out = tmp_path / "out"
    mine.save_pretrained(str(out))
    back = transformers.Qwen2VLForConditionalGeneration.from_pretrained(str(out), torch_dtype=torch.float32).eval()
    with torch.no_grad():
        torch.testing.assert_close(back(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits, want,
                                   rtol=3e-4, atol=3e-4)


def test_image_processor_matches_hugging_face_and_vl_training_step():
    import numpy as np

    from paddleformers_b200.models.vision_language import Qwen2VLConfig, Qwen2VLForConditionalGeneration, mm_collate_fn
    from paddleformers_b200.transformers.image_processing import Qwen2VLImageProcessor, smart_resize

    rng = np.random.RandomState(0)
    imgs = [(rng.rand(37, 50, 3) * 255).astype("uint8"), (rng.rand(20, 90, 3) * 255).astype("uint8")]
    kw = dict(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=16 * 16, max_pixels=64 * 64)
    mine = Qwen2VLImageProcessor(**kw)(imgs)
    try:
        ref = transformers.Qwen2VLImageProcessor(**kw)(images=imgs, return_tensors="pt")
    except Exception as e:  # noqa: BLE001 - optional image backend missing
        pytest.skip(f"transformers image processor unavailable: {e}")
    assert torch.equal(mine["image_grid_thw"], ref["image_grid_thw"])
    torch.testing.assert_close(mine["pixel_values"], ref["pixel_values"].float(), rtol=1e-4, atol=2e-2)
    assert smart_resize(37, 50, 8, 256, 4096) == (40, 48)
    # a few optimisation steps on image + text examples: the loss falls and the vision tower receives gradients
    torch.manual_seed(0)
    cfg = Qwen2VLConfig(text_config=dict(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2,
                                         num_key_value_heads=1, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}),
                        vision_config=dict(depth=1, embed_dim=16, hidden_size=32, mlp_ratio=2, num_heads=2, patch_size=4),
                        image_token_id=60)
    model = Qwen2VLForConditionalGeneration(cfg, dtype=torch.float32)
    proc = Qwen2VLImageProcessor(**kw)
    examples = []
    for im in imgs:
        out = proc([im])
        n = proc.num_image_tokens(out["image_grid_thw"][0])
        ids = [1, 2] + [60] * n + [3, 4, 5, 6]
        labels = [-100] * (2 + n) + [4, 5, 6, -100]
        examples.append({"input_ids": ids, "labels": labels, **out})
    # one example per forward: placeholders of a row must match that row's images
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    losses = []
    for _ in range(6):
        total = 0.0
        for ex in examples:
            batch = mm_collate_fn([ex])
            loss = model(**batch).loss
            opt.zero_grad()
            loss.backward()
            opt.step()
            total += loss.item()
        losses.append(total)
    assert losses[-1] < losses[0]
    assert model.visual.patch_embed.weight.grad is not None and model.visual.patch_embed.weight.grad.abs().sum() > 0


def test_qwen2_5_vl_matches_hugging_face(tmp_path):
    """Windowed vision attention (window re-ordering and its inverse), RMSNorm / SwiGLU vision blocks."""
    if not hasattr(transformers, "Qwen2_5_VLForConditionalGeneration"):
        pytest.skip("transformers has no Qwen2.5-VL")
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(6)
    vc = dict(depth=3, hidden_size=32, intermediate_size=48, num_heads=2, in_chans=3, out_hidden_size=64, patch_size=4,
              spatial_merge_size=2, temporal_patch_size=2, window_size=16, fullatt_block_indexes=[1], hidden_act="silu",
              tokens_per_second=1)      # still images: the temporal position of an image is the position where it starts
    tc = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              max_position_embeddings=128, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, tie_word_embeddings=False)
    cfg = transformers.Qwen2_5_VLConfig(text_config=tc, vision_config=vc, image_token_id=120, video_token_id=121,
                                        vision_start_token_id=118, vision_end_token_id=119)
    hf = transformers.Qwen2_5_VLForConditionalGeneration(cfg).eval().float()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    grid = torch.tensor([[1, 6, 10], [1, 4, 4]])                      # 60 and 16 patches -> 15 and 4 tokens; windows of 2 x 2 groups
    pixels = torch.randn(int(grid.prod(-1).sum()), 3 * 2 * 4 * 4)
    with torch.no_grad():
        torch.testing.assert_close(mine.visual(pixels, grid), hf.model.visual(pixels, grid_thw=grid).pooler_output, rtol=1e-4, atol=1e-5)
    ids = torch.tensor([[5, 118] + [120] * 15 + [119, 7, 8, 118] + [120] * 4 + [119, 10, 11]])
    types = (ids == 120).int()
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits
        got = mine(ids, pixel_values=pixels, image_grid_thw=grid, return_logits=True).logits
    torch.testing.assert_close(got, want, rtol=3e-4, atol=3e-4)


def test_internlm2_checkpoint_layout_against_a_llama_oracle(tmp_path):
    """InternLM2 is a Llama whose checkpoint uses other names and a fused ``wqkv`` grouped by kv head. A Hugging Face Llama is
    rewritten into that format by hand (independently of the framework's rules); loading it must reproduce the Llama's logits,
    and saving must reproduce the rewritten tensors exactly."""
    import json

    from safetensors.torch import load_file, save_file

    torch.manual_seed(0)
    hf_cfg = transformers.LlamaConfig(**{**BASE, "rope_theta": 10000.0})
    hf = transformers.LlamaForCausalLM(hf_cfg).eval().float()
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    Hq, Hkv, D = 4, 2, 16
    out = {"model.tok_embeddings.weight": sd["model.embed_tokens.weight"], "model.norm.weight": sd["model.norm.weight"],
           "output.weight": sd["lm_head.weight"]}
    for i in range(2):
        p, q = f"model.layers.{i}.", f"model.layers.{i}."
        wq = sd[p + "self_attn.q_proj.weight"].view(Hkv, Hq // Hkv, D, -1)
        wk = sd[p + "self_attn.k_proj.weight"].view(Hkv, 1, D, -1)
        wv = sd[p + "self_attn.v_proj.weight"].view(Hkv, 1, D, -1)
        out[q + "attention.wqkv.weight"] = torch.cat([wq, wk, wv], dim=1).reshape(-1, wq.shape[-1]).contiguous()
        out[q + "attention.wo.weight"] = sd[p + "self_attn.o_proj.weight"]
        out[q + "attention_norm.weight"] = sd[p + "input_layernorm.weight"]
        out[q + "ffn_norm.weight"] = sd[p + "post_attention_layernorm.weight"]
        out[q + "feed_forward.w1.weight"] = sd[p + "mlp.gate_proj.weight"]
        out[q + "feed_forward.w3.weight"] = sd[p + "mlp.up_proj.weight"]
        out[q + "feed_forward.w2.weight"] = sd[p + "mlp.down_proj.weight"]
    src = tmp_path / "src"
    src.mkdir()
    save_file({k: v.contiguous() for k, v in out.items()}, str(src / "model.safetensors"), metadata={"format": "pt"})
    cfg = {k: v for k, v in hf_cfg.to_dict().items() if k in BASE or k in ("rms_norm_eps", "rope_theta", "head_dim", "hidden_act")}
    cfg.update(model_type="internlm2", bias=False, rope_theta=10000.0)
    (src / "config.json").write_text(json.dumps(cfg))
    mine = AutoModelForCausalLM.from_pretrained(str(src), dtype=torch.float32).eval()
    ids = torch.randint(0, 128, (2, 24))
    with torch.no_grad():
        torch.testing.assert_close(mine(ids, return_logits=True).logits, hf(input_ids=ids).logits, rtol=2e-4, atol=2e-4)
    mine.save_pretrained(str(tmp_path / "out"))
    back = load_file(str(tmp_path / "out" / "model.safetensors"))
    assert set(back) == set(out)
    for k in out:
        assert torch.equal(back[k], out[k]), k


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_vl_matches_hugging_face(tmp_path, moe):
    """Interpolated position embeddings, deepstack features added after the first decoder layers, interleaved multimodal rotary
    sections and per-head QK norm against ``transformers``' Qwen3-VL, on two images of different sizes between text tokens."""
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    names = ("Qwen3VLMoeConfig", "Qwen3VLMoeForConditionalGeneration") if moe else ("Qwen3VLConfig", "Qwen3VLForConditionalGeneration")
    if not all(hasattr(transformers, n) for n in names):
        pytest.skip("transformers has no Qwen3-VL")
    HFConfig, HFModel = (getattr(transformers, n) for n in names)
    torch.manual_seed(7)
    vc = dict(depth=3, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4, spatial_merge_size=2,
              temporal_patch_size=2, out_hidden_size=64, num_position_embeddings=36, deepstack_visual_indexes=[0, 2])
    tc = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, max_position_embeddings=128, tie_word_embeddings=False,
              rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [4, 2, 2], "mrope_interleaved": True})
    if moe:
        tc.update(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24, decoder_sparse_step=1, mlp_only_layers=[1])
    cfg = HFConfig(text_config=tc, vision_config=vc, image_token_id=120, video_token_id=121,
                                     vision_start_token_id=118, vision_end_token_id=119)
    hf = HFModel(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.normal_(1.0 if "norm" in n and "bias" not in n else 0.0, 0.1)
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    grid = torch.tensor([[1, 4, 6], [1, 2, 2]])
    pixels = torch.randn(int(grid.prod(-1).sum()), 3 * 2 * 4 * 4)
    ids = torch.tensor([[5, 6, 118] + [120] * 6 + [119, 7, 8, 9, 118, 120, 119, 10, 11]])
    types = (ids == 120).int()
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits
        got = mine(ids, pixel_values=pixels, image_grid_thw=grid, return_logits=True).logits
    torch.testing.assert_close(got, want, rtol=3e-4, atol=3e-4)
    text = torch.randint(0, 100, (2, 12))
    with torch.no_grad():
        torch.testing.assert_close(mine(text, return_logits=True).logits, hf(input_ids=text).logits, rtol=3e-4, atol=3e-4)
    out = tmp_path / "out"
    mine.save_pretrained(str(out))
    back = HFModel.from_pretrained(str(out), torch_dtype=torch.float32).eval()
    with torch.no_grad():
        torch.testing.assert_close(back(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits, want,
                                   rtol=3e-4, atol=3e-4)
    # gradients reach the vision tower, its position table and the deepstack mergers
    mine.train()
    mine(ids, pixel_values=pixels, image_grid_thw=grid, labels=torch.roll(ids, -1, 1)).loss.backward()
    for name in ("visual.pos_embed.weight", "visual.deepstack_mergers.1.fc2.weight", "visual.blocks.0.qkv.weight"):
        assert dict(mine.named_parameters())[name].grad.abs().sum() > 0, name


def test_video_processor_patch_layout_and_model_consumes_it():
    """A clip goes through the video processor and the Qwen2-VL model; the patch layout is checked against the image processor
    (a clip of identical frames equals the still image repeated over time) and against ``transformers`` when its video
    processor is importable."""
    import numpy as np

    from paddleformers_b200.models.vision_language import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    from paddleformers_b200.transformers.image_processing import Qwen2VLImageProcessor, Qwen2VLVideoProcessor

    rng = np.random.RandomState(0)
    kw = dict(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=16 * 16, max_pixels=64 * 64)
    frame = (rng.rand(24, 32, 3) * 255).astype("uint8")
    vp = Qwen2VLVideoProcessor(**kw, min_frames=2)
    still = Qwen2VLImageProcessor(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=16 * 16, max_pixels=32 * 32)([frame])
    clip = np.stack([frame] * 2)
    out = vp([clip])
    assert out["video_grid_thw"].tolist() == [[1, 6, 8]] and torch.equal(out["video_grid_thw"][0, 1:], still["image_grid_thw"][0, 1:])
    torch.testing.assert_close(out["pixel_values_videos"], still["pixel_values"])
    # 5 distinct frames: padded to 6 by repeating the last one -> 3 temporal patches; sampling picks evenly spaced frames
    clip5 = (rng.rand(5, 24, 32, 3) * 255).astype("uint8")
    o5 = vp([clip5])
    assert o5["video_grid_thw"][0, 0] == 3 and o5["pixel_values_videos"].shape == (3 * int(o5["video_grid_thw"][0, 1:].prod()), 3 * 2 * 16)
    assert vp.sample_indices(30, num_frames=4).tolist() == [0, 10, 19, 29]
    assert len(vp.sample_indices(300, fps=2.0, source_fps=30.0)) == 20
    try:
        ref = transformers.Qwen2VLVideoProcessor(patch_size=4, merge_size=2, temporal_patch_size=2, min_pixels=16 * 16, max_pixels=64 * 64,
                                                 do_sample_frames=False)(videos=[torch.from_numpy(clip5).permute(0, 3, 1, 2)],
                                                                         return_tensors="pt")
        if ref["video_grid_thw"].tolist() == o5["video_grid_thw"].tolist():
            torch.testing.assert_close(o5["pixel_values_videos"], ref["pixel_values_videos"].float(), rtol=1e-3, atol=5e-2)
    except Exception:  # noqa: BLE001 - optional backend (torchvision) or a different resize budget rule
        pass
    torch.manual_seed(0)
    cfg = Qwen2VLConfig(text_config=dict(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2,
                                         num_key_value_heads=1, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}),
                        vision_config=dict(depth=1, embed_dim=16, hidden_size=32, mlp_ratio=2, num_heads=2, patch_size=4),
                        image_token_id=60, video_token_id=61)
    model = Qwen2VLForConditionalGeneration(cfg, dtype=torch.float32)
    n_tok = int(o5["video_grid_thw"][0].prod()) // 4
    ids = torch.tensor([[1, 2] + [61] * n_tok + [3, 4]])
    out = model(ids, pixel_values_videos=o5["pixel_values_videos"], video_grid_thw=o5["video_grid_thw"], labels=torch.roll(ids, -1, 1))
    out.loss.backward()
    assert torch.isfinite(out.loss) and model.visual.patch_embed.weight.grad.abs().sum() > 0


def test_gemma2_capped_loss_and_cached_decoding_match_hugging_face(tmp_path):
    """Soft-capped scores and logits take the unfused paths: the loss (head, cap, cross entropy in token chunks) and greedy
    decoding with the key / value cache still agree with ``transformers``."""
    from paddleformers_b200.generation.utils import GenerationConfig, generate

    torch.manual_seed(2)
    cfg = transformers.Gemma2Config(**{**BASE, "head_dim": 16, "num_hidden_layers": 2, "sliding_window": 6, "query_pre_attn_scalar": 24,
                                       "attn_logit_softcapping": 5.0, "final_logit_softcapping": 3.0, "tie_word_embeddings": True})
    hf = transformers.Gemma2ForCausalLM(cfg).float()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    mine = AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32)
    ids = torch.randint(1, 128, (2, 20))
    labels = torch.cat([ids[:, 1:], torch.full((2, 1), -100)], dim=1)
    out = mine(ids, labels=labels)
    want = hf(input_ids=ids, labels=ids)
    assert out.loss.item() == pytest.approx(want.loss.item(), rel=1e-5)
    out.loss.backward()
    want.loss.backward()
    torch.testing.assert_close(mine.model.embed_tokens.weight.grad, hf.model.embed_tokens.weight.grad, rtol=1e-4, atol=1e-6)
    mine.eval(); hf.eval()
    got = generate(mine, ids[:, :8], GenerationConfig(max_new_tokens=6))
    ref = hf.generate(ids[:, :8], max_new_tokens=6, do_sample=False, pad_token_id=0)
    assert torch.equal(got, ref[:, :got.shape[1]])


def test_gpt_oss_mxfp4_checkpoint_loads_through_the_virtual_tensors(tmp_path):
    """The released gpt-oss checkpoints keep the expert matrices as MXFP4 blocks + scales. A Hugging Face model whose expert
    weights are exactly representable in MXFP4 is rewritten into that format; loading it must reproduce the logits."""
    import json

    from safetensors.torch import load_file, save_file

    from paddleformers_b200.quantization.checkpoint_dequant import dequant_mxfp4, quant_mxfp4

    torch.manual_seed(4)
    cfg = transformers.GptOssConfig(**{**BASE, "head_dim": 16, "intermediate_size": 32, "num_hidden_layers": 2, "num_local_experts": 4,
                                       "num_experts_per_tok": 2, "sliding_window": 8,
                                       "rope_parameters": {"rope_type": "default", "rope_theta": 10000.0}})
    hf = transformers.GptOssForCausalLM(cfg).eval().float()
    with torch.no_grad():                       # snap the expert matrices onto the MXFP4 grid (quantised along the input dimension)
        for n, p in hf.named_parameters():
            if n.endswith("experts.gate_up_proj") or n.endswith("experts.down_proj"):
                t = (p * 8).transpose(1, 2).contiguous()                         # [E, out, in]
                p.copy_(dequant_mxfp4(*quant_mxfp4(t), torch.float32).transpose(1, 2))
    hf.save_pretrained(str(tmp_path / "plain"), safe_serialization=True)
    sd = load_file(str(tmp_path / "plain" / "model.safetensors"))
    out = {}
    for k, v in sd.items():
        if k.endswith("experts.gate_up_proj") or k.endswith("experts.down_proj"):
            blocks, scales = quant_mxfp4(v.float().transpose(1, 2).contiguous())
            out[k + "_blocks"], out[k + "_scales"] = blocks, scales
        else:
            out[k] = v
    q = tmp_path / "mxfp4"
    q.mkdir()
    save_file({k: v.contiguous() for k, v in out.items()}, str(q / "model.safetensors"), metadata={"format": "pt"})
    conf = json.loads((tmp_path / "plain" / "config.json").read_text())
    conf["quantization_config"] = {"quant_method": "mxfp4", "modules_to_not_convert": ["model.layers.*.self_attn", "lm_head"]}
    (q / "config.json").write_text(json.dumps(conf))
    mine = AutoModelForCausalLM.from_pretrained(str(q), dtype=torch.float32).eval()
    ids = torch.randint(0, 128, (2, 20))
    with torch.no_grad():
        torch.testing.assert_close(mine(ids, return_logits=True).logits, hf(input_ids=ids).logits, rtol=2e-4, atol=2e-4)


def test_glm4v_moe_matches_hugging_face(tmp_path):
    """GLM-4.5V: bicubic position-embedding samples, strided-convolution patch merge, gated merger, multimodal rotary sections on
    the rotated half of each head, GLM-4.5 MoE decoder with biases, against ``transformers`` on two images between text tokens."""
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    if not hasattr(transformers, "Glm4vMoeForConditionalGeneration"):
        pytest.skip("transformers has no GLM-4.5V")
    torch.manual_seed(11)
    vc = dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, image_size=24, patch_size=4, spatial_merge_size=2,
              temporal_patch_size=2, out_hidden_size=64)
    tc = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, max_position_embeddings=128, tie_word_embeddings=False, moe_intermediate_size=32, n_routed_experts=4,
              num_experts_per_tok=2, n_shared_experts=1, first_k_dense_replace=1, n_group=1, topk_group=1,
              rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5, "mrope_section": [2, 1, 1]})
    cfg = transformers.Glm4vMoeConfig(text_config=tc, vision_config=vc, image_token_id=120, video_token_id=121,
                                      image_start_token_id=118, image_end_token_id=119)
    hf = transformers.Glm4vMoeForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.normal_(1.0 if "norm" in n and "bias" not in n else 0.0, 0.1)
        for n, b in hf.named_buffers():
            if "e_score_correction_bias" in n:
                b.normal_(0.0, 0.1)
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    grid = torch.tensor([[1, 4, 6], [1, 2, 2]])
    pixels = torch.randn(int(grid.prod(-1).sum()), 3 * 2 * 4 * 4)
    ids = torch.tensor([[5, 6, 118] + [120] * 6 + [119, 7, 8, 9, 118, 120, 119, 10, 11]])
    types = (ids == 120).int()
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits
        got = mine(ids, pixel_values=pixels, image_grid_thw=grid, return_logits=True).logits
    torch.testing.assert_close(got, want, rtol=3e-4, atol=3e-4)
    out = tmp_path / "out"
    mine.save_pretrained(str(out))
    back = transformers.Glm4vMoeForConditionalGeneration.from_pretrained(str(out), torch_dtype=torch.float32).eval()
    with torch.no_grad():
        torch.testing.assert_close(back(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits, want,
                                   rtol=3e-4, atol=3e-4)


@pytest.mark.parametrize("use_head", [True, False])
def test_siglip_vision_tower_matches_hugging_face(tmp_path, use_head):
    """Hidden states and the probe-attention pooled vector, loaded from a checkpoint written by transformers; a checkpoint
    written here loads back into transformers with identical outputs."""
    from transformers import SiglipVisionConfig as HFConfig, SiglipVisionModel as HFModel

    from paddleformers_b200.transformers.auto import AutoModel

    torch.manual_seed(0)
    hf = HFModel(HFConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=32,
                          patch_size=8, vision_use_head=use_head)).eval()
    hf.save_pretrained(tmp_path / "hf")
    mine = AutoModel.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    x = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        want = hf(pixel_values=x)
        hidden, pooled = mine(x)
    assert (want.last_hidden_state - hidden).abs().max() < 1e-4
    if use_head:
        assert (want.pooler_output - pooled).abs().max() < 1e-4
    else:
        assert pooled is None
    mine.save_pretrained(str(tmp_path / "mine"))
    back = HFModel.from_pretrained(tmp_path / "mine").eval()
    with torch.no_grad():
        again = back(pixel_values=x)
    assert (again.last_hidden_state - want.last_hidden_state).abs().max() < 1e-5


def test_paligemma_matches_hugging_face(tmp_path):
    """SigLIP tower + projector + Gemma decoder with two-way attention on the prefix: logits under the training mask
    (prefix from ``token_type_ids``, different prefix lengths per row) and under the prompt mask (everything two-way), the loss on
    the suffix, and a checkpoint written here read back by transformers."""
    from transformers import PaliGemmaConfig as HFConfig, PaliGemmaForConditionalGeneration as HFModel

    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(0)
    hf = HFModel(HFConfig(
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, image_size=16, patch_size=8,
                           projection_dim=64, vision_use_head=False),
        text_config=dict(model_type="gemma", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=1, head_dim=16, vocab_size=300),
        image_token_id=299, hidden_size=64, projection_dim=64))
    hf.save_pretrained(tmp_path / "hf")
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    ids = torch.tensor([[299] * 4 + [2, 5, 6, 7, 8, 9, 10, 11], [299] * 4 + [2, 15, 16, 17, 18, 19, 20, 21]])
    types = torch.tensor([[0] * 8 + [1] * 4, [0] * 6 + [1] * 6])
    pixels = torch.randn(2, 3, 16, 16)
    labels = torch.where(types == 1, ids, torch.full_like(ids, -100))
    shifted = torch.cat([labels[:, 1:], torch.full_like(labels[:, :1], -100)], dim=1)     # transformers shifts inside the model
    with torch.no_grad():
        hf.train()                                   # the training mask is only built in training mode
        want = hf(input_ids=ids, pixel_values=pixels, token_type_ids=types, labels=labels)
        hf.eval()
        got = mine(ids, pixel_values=pixels, token_type_ids=types, labels=shifted, return_logits=True)
        assert (want.logits - got.logits).abs().max() < 1e-4
        assert abs(want.loss.item() - got.loss.item()) < 1e-4
        causal = mine.language(ids).logits           # the same decoder without the two-way prefix must differ on prefix rows
        assert (causal[:, 4:6] - got.logits[:, 4:6]).abs().max() > 1e-3
        want_prompt = hf(input_ids=ids, pixel_values=pixels)
        got_prompt = mine(ids, pixel_values=pixels)
        assert (want_prompt.logits - got_prompt.logits).abs().max() < 1e-4
    out = mine(ids, pixel_values=pixels, token_type_ids=types, labels=shifted)
    out.loss.backward()
    assert mine.projector.weight.grad.abs().sum() > 0 and mine.vision_tower.patch_embedding.weight.grad.abs().sum() > 0
    mine.save_pretrained(str(tmp_path / "mine"))
    back = HFModel.from_pretrained(tmp_path / "mine").eval()
    with torch.no_grad():
        again = back(input_ids=ids, pixel_values=pixels)
    assert (again.logits - want_prompt.logits).abs().max() < 1e-5


def test_paligemma2_window_layers_keep_the_prefix_whole(tmp_path):
    """Gemma 2 decoder (soft-capped scores, alternating sliding-window layers) under a prefix longer than the window: a
    window never cuts through the two-way prefix, and suffix rows see the usual window."""
    from transformers import PaliGemmaConfig as HFConfig, PaliGemmaForConditionalGeneration as HFModel

    from paddleformers_b200.models.paligemma import two_way_block_ends, two_way_block_starts
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    blocks = torch.tensor([[1, 1, 1, 0, 0, 1, 1, 0], [0, 1, 1, 1, 1, 0, 0, 0]]).bool()
    assert two_way_block_starts(blocks).tolist() == [[0, 0, 0, 3, 4, 5, 5, 7], [0, 1, 1, 1, 1, 5, 6, 7]]
    assert two_way_block_ends(blocks).tolist() == [[3, 3, 3, 0, 0, 7, 7, 0], [0, 5, 5, 5, 5, 0, 0, 0]]
    torch.manual_seed(0)
    hf = HFModel(HFConfig(
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, image_size=16, patch_size=8,
                           projection_dim=64, vision_use_head=False),
        text_config=dict(model_type="gemma2", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=1, head_dim=16, vocab_size=300, sliding_window=4, query_pre_attn_scalar=16),
        image_token_id=299, hidden_size=64, projection_dim=64))
    hf.save_pretrained(tmp_path)
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    ids = torch.tensor([[299] * 4 + [2, 5, 6, 7, 8, 9, 10, 11, 12, 13], [299] * 4 + [2, 15, 16, 17, 18, 19, 20, 21, 22, 23]])
    types = torch.tensor([[0] * 8 + [1] * 6, [0] * 6 + [1] * 8])
    pixels = torch.randn(2, 3, 16, 16)
    with torch.no_grad():
        hf.train()
        want = hf(input_ids=ids, pixel_values=pixels, token_type_ids=types, labels=ids).logits
        got = mine(ids, pixel_values=pixels, token_type_ids=types).logits
    assert (want - got).abs().max() < 5e-4


def test_gemma3_with_images_matches_hugging_face(tmp_path):
    """Two images in one row: pooled + normalised + projected SigLIP features, two-way attention inside each image on global and
    on sliding-window layers (window shorter than an image block), causal text."""
    from transformers import Gemma3Config as HFConfig, Gemma3ForConditionalGeneration as HFModel

    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(0)
    hf = HFModel(HFConfig(
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, image_size=32, patch_size=8,
                           vision_use_head=False),
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=1,
                         head_dim=16, vocab_size=300, sliding_window=3, query_pre_attn_scalar=16,
                         layer_types=["sliding_attention", "full_attention", "sliding_attention"]),
        mm_tokens_per_image=4, image_token_index=299, boi_token_index=297, eoi_token_index=298)).eval()
    with torch.no_grad():
        hf.model.multi_modal_projector.mm_input_projection_weight.normal_(0, 0.1)
        hf.model.multi_modal_projector.mm_soft_emb_norm.weight.normal_(0, 0.1)
    hf.save_pretrained(tmp_path / "hf")
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    ids = torch.tensor([[2, 5, 297] + [299] * 4 + [298, 6, 297] + [299] * 4 + [298, 7, 8, 9, 10]])
    types = (ids == 299).long()
    pixels = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, token_type_ids=types).logits
        got = mine(ids, pixel_values=pixels).logits                      # types default to the image placeholders
        assert (want - got).abs().max() < 1e-4
        assert (mine(ids, pixel_values=pixels, token_type_ids=types).logits - got).abs().max() == 0
    labels = torch.cat([ids[:, 1:], torch.full_like(ids[:, :1], -100)], dim=1).masked_fill(ids.roll(-1, 1) >= 297, -100)
    mine(ids, pixel_values=pixels, labels=labels).loss.backward()
    assert mine.mm_input_projection_weight.grad.abs().sum() > 0
    mine.save_pretrained(str(tmp_path / "mine"))
    back = HFModel.from_pretrained(tmp_path / "mine").eval()
    with torch.no_grad():
        assert (back(input_ids=ids, pixel_values=pixels, token_type_ids=types).logits - want).abs().max() < 1e-5
    fresh = AutoModelForConditionalGeneration.from_config(mine.config, dtype=torch.float32)
    assert fresh.mm_input_projection_weight.abs().sum() > 0


def test_aya_vision_matches_hugging_face(tmp_path):
    """SigLIP features of the last encoder block (no final LayerNorm), 2 x 2 patches folded into channels, LayerNorm + SwiGLU
    projector, Cohere 2 decoder with sliding-window layers."""
    from transformers import AyaVisionConfig as HFConfig, AyaVisionForConditionalGeneration as HFModel

    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(0)
    hf = HFModel(HFConfig(
        vision_config=dict(model_type="siglip_vision_model", hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                           num_attention_heads=2, image_size=32, patch_size=8, vision_use_head=False),
        text_config=dict(model_type="cohere2", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=1, head_dim=16, vocab_size=300, sliding_window=4),
        downsample_factor=2, alignment_intermediate_size=96, image_token_index=299)).eval()
    hf.save_pretrained(tmp_path / "hf")
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    ids = torch.tensor([[2, 5] + [299] * 4 + [6, 7, 8, 9, 10], [2] + [299] * 4 + [6, 7, 8, 9, 10, 11]])
    pixels = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels).logits
        assert (want - mine(ids, pixel_values=pixels).logits).abs().max() < 1e-4
    mine.save_pretrained(str(tmp_path / "mine"))
    back = HFModel.from_pretrained(tmp_path / "mine").eval()
    with torch.no_grad():
        assert (back(input_ids=ids, pixel_values=pixels).logits - want).abs().max() < 1e-5


def test_shieldgemma2_classifier_matches_hugging_face(tmp_path):
    from transformers import ShieldGemma2Config as HFConfig, ShieldGemma2ForImageClassification as HFModel

    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(0)
    hf = HFModel(HFConfig(
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, image_size=32, patch_size=8,
                           vision_use_head=False),
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
                         head_dim=16, vocab_size=300, sliding_window=3, query_pre_attn_scalar=16),
        mm_tokens_per_image=4, image_token_index=299, boi_token_index=297, eoi_token_index=298, yes_token_index=11, no_token_index=12)).eval()
    with torch.no_grad():
        hf.model.model.multi_modal_projector.mm_input_projection_weight.normal_(0, 0.1)
    hf.save_pretrained(tmp_path / "hf")
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    ids = torch.tensor([[2, 297] + [299] * 4 + [298, 6, 7, 8, 9]])
    pixels = torch.randn(1, 3, 32, 32)
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, token_type_ids=(ids == 299).long())
        got = mine(ids, pixel_values=pixels)
    assert (want.probabilities - got.probabilities).abs().max() < 1e-5 and (want.logits - got.logits).abs().max() < 1e-4
    mine.save_pretrained(str(tmp_path / "mine"))
    back = HFModel.from_pretrained(tmp_path / "mine").eval()
    with torch.no_grad():
        again = back(input_ids=ids, pixel_values=pixels, token_type_ids=(ids == 299).long())
    assert (again.logits - want.logits).abs().max() < 1e-5


def test_whisper_matches_hugging_face(tmp_path):
    """Encoder-decoder speech model: logits and loss under teacher forcing (decoder fed the labels shifted right), checkpoint
    round trip, and greedy decoding consistent with the teacher-forced argmax."""
    from transformers import WhisperConfig as HFConfig, WhisperForConditionalGeneration as HFModel

    from paddleformers_b200.transformers.auto import AutoModelForSpeechSeq2Seq

    torch.manual_seed(0)
    hf = HFModel(HFConfig(vocab_size=120, num_mel_bins=8, encoder_layers=2, encoder_attention_heads=2, decoder_layers=2,
                          decoder_attention_heads=2, decoder_ffn_dim=64, encoder_ffn_dim=64, d_model=32, max_source_positions=20,
                          max_target_positions=24, decoder_start_token_id=1, pad_token_id=0, bos_token_id=2, eos_token_id=3,
                          suppress_tokens=None, begin_suppress_tokens=None)).eval()
    hf.save_pretrained(tmp_path / "hf")
    mine = AutoModelForSpeechSeq2Seq.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    feats = torch.randn(2, 8, 40)
    labels = torch.randint(4, 120, (2, 9))
    labels[1, 6:] = -100
    with torch.no_grad():
        want = hf(input_features=feats, labels=labels)
        got = mine(feats, labels=labels, return_logits=True)
    assert (want.logits - got.logits).abs().max() < 1e-4 and abs(want.loss.item() - got.loss.item()) < 1e-4
    mine(feats, labels=labels).loss.backward()
    assert mine.model.encoder.conv1.weight.grad.abs().sum() > 0 and mine.model.encoder.embed_positions.weight.grad is None
    out = mine.generate(feats, max_new_tokens=5)
    with torch.no_grad():
        step = hf(input_features=feats, decoder_input_ids=out[:, :-1]).logits.argmax(-1)
    assert out.shape == (2, 6) and torch.equal(step[:, -1], out[:, -1]) and torch.equal(step[:, 0], out[:, 1])
    mine.save_pretrained(str(tmp_path / "mine"))
    back = HFModel.from_pretrained(tmp_path / "mine").eval()
    with torch.no_grad():
        assert (back(input_features=feats, labels=labels).logits - want.logits).abs().max() < 1e-5


def test_log_mel_features_match_hugging_face(tmp_path):
    import numpy as np
    from transformers import WhisperFeatureExtractor as HFExtractor

    from paddleformers_b200.transformers.audio_processing import LogMelFeatureExtractor

    hf, mine = HFExtractor(feature_size=80, chunk_length=2), LogMelFeatureExtractor(feature_size=80, chunk_length=2)
    assert np.abs(hf.mel_filters - mine.mel_filters.numpy()).max() < 1e-6
    rng = np.random.default_rng(0)
    waves = [rng.standard_normal(20000).astype(np.float32) * 0.1, np.sin(np.arange(40000) * 0.05).astype(np.float32)]
    want = hf(waves, sampling_rate=16000, return_tensors="pt")["input_features"]
    got = mine(waves, sampling_rate=16000)["input_features"]
    assert got.shape == want.shape == (2, 80, 200) and (want - got).abs().max() < 1e-4
    mine.save_pretrained(str(tmp_path))
    again = LogMelFeatureExtractor.from_pretrained(str(tmp_path))
    assert again.nb_max_frames == 200 and torch.equal(again(waves)["input_features"], got)
    with pytest.raises(ValueError, match="resample"):
        mine(waves, sampling_rate=8000)


def test_glm4_dense_and_glm_ocr_match_hugging_face(tmp_path):
    """GLM-4 dense text (four norms per block, interleaved partial rotary rows, fused gate_up in the checkpoint) and GLM-OCR on top
    of it (vision tower with per-head q / k norms and no position table), against ``transformers`` both ways."""
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(3)
    hf_text = transformers.Glm4ForCausalLM(transformers.Glm4Config(
        vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
        attention_bias=True, pad_token_id=0)).eval()
    hf_text.save_pretrained(str(tmp_path / "glm4"))
    text = AutoModelForCausalLM.from_pretrained(str(tmp_path / "glm4"), dtype=torch.float32).eval()
    tokens = torch.randint(0, 300, (2, 12))
    with torch.no_grad():
        torch.testing.assert_close(text(tokens).logits, hf_text(tokens).logits, rtol=1e-4, atol=1e-4)
    text.save_pretrained(str(tmp_path / "glm4_back"))
    with torch.no_grad():
        torch.testing.assert_close(transformers.Glm4ForCausalLM.from_pretrained(str(tmp_path / "glm4_back")).eval()(tokens).logits,
                                   hf_text(tokens).logits, rtol=1e-5, atol=1e-5)

    if not hasattr(transformers, "GlmOcrForConditionalGeneration"):
        pytest.skip("transformers has no GLM-OCR")
    vc = dict(hidden_size=32, depth=2, num_heads=2, out_hidden_size=48, intermediate_size=64, image_size=32, patch_size=4,
              spatial_merge_size=2, temporal_patch_size=2)
    tc = dict(vocab_size=300, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [2, 1, 1],
                                            "partial_rotary_factor": 0.5})
    hf = transformers.GlmOcrForConditionalGeneration(transformers.GlmOcrConfig(
        vision_config=vc, text_config=tc, image_token_id=299, video_token_id=298, image_start_token_id=297, image_end_token_id=296)).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if p.dim() == 1:
                p.normal_(1.0 if "norm" in n and "bias" not in n else 0.0, 0.1)
    hf.save_pretrained(str(tmp_path / "ocr"))
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "ocr"), dtype=torch.float32).eval()
    grid = torch.tensor([[1, 4, 6], [1, 2, 2]])
    pixels = torch.randn(int(grid.prod(-1).sum()), 3 * 2 * 4 * 4)
    ids = torch.tensor([[5, 6, 297] + [299] * 6 + [296, 7, 8, 9, 297, 299, 296, 10, 11]])
    types = (ids == 299).int()
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits
        got = mine(ids, pixel_values=pixels, image_grid_thw=grid, return_logits=True).logits
    torch.testing.assert_close(got, want, rtol=3e-4, atol=3e-4)
    mine.save_pretrained(str(tmp_path / "ocr_back"))
    back = transformers.GlmOcrForConditionalGeneration.from_pretrained(str(tmp_path / "ocr_back")).eval()
    with torch.no_grad():
        torch.testing.assert_close(back(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits, want,
                                   rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("family", ["paligemma", "gemma3"])
def test_greedy_generation_of_siglip_composites_matches_hugging_face(tmp_path, family):
    """Decoding without a cache under the training masks (two-way prompt / image blocks, causal continuation) gives the tokens
    that transformers produces with its cache."""
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(5)
    vision = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, image_size=16, patch_size=8, vision_use_head=False)
    text = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=16,
                vocab_size=300, initializer_range=0.3)
    if family == "paligemma":
        hf = transformers.PaliGemmaForConditionalGeneration(transformers.PaliGemmaConfig(
            vision_config=dict(vision, projection_dim=64), text_config=dict(text, model_type="gemma"), image_token_id=299, hidden_size=64,
            projection_dim=64)).eval()
        ids = torch.tensor([[299] * 4 + [2, 5, 6, 7]])
        extra = {}
    else:
        hf = transformers.Gemma3ForConditionalGeneration(transformers.Gemma3Config(
            vision_config=vision, text_config=dict(text, sliding_window=4, query_pre_attn_scalar=16), mm_tokens_per_image=4,
            image_token_index=299, boi_token_index=297, eoi_token_index=298)).eval()
        with torch.no_grad():
            hf.model.multi_modal_projector.mm_input_projection_weight.normal_(0, 0.3)
        ids = torch.tensor([[2, 297] + [299] * 4 + [298, 5, 6, 7]])
        extra = {"token_type_ids": (ids == 299).long()}
    hf.generation_config.eos_token_id = None
    hf.save_pretrained(str(tmp_path))
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path), dtype=torch.float32).eval()
    pixels = torch.randn(1, 3, 16, 16)
    want = hf.generate(input_ids=ids, pixel_values=pixels, max_new_tokens=6, do_sample=False, **extra)
    got = mine.generate(ids, pixel_values=pixels, max_new_tokens=6, eos_token_id=-1)
    assert got.tolist() == want.tolist()
    with torch.no_grad():                                        # the step after the last one, by logits (tiny tied models repeat tokens)
        types = {"token_type_ids": torch.cat([torch.zeros_like(ids), torch.ones_like(want[:, ids.shape[1]:])], 1)} if family == "paligemma" \
            else {"token_type_ids": (want == 299).long()}
        hf.train()
        ref = hf(input_ids=want, pixel_values=pixels, labels=want, **types).logits[:, -1]
        hf.eval()
        mine_types = types if family == "paligemma" else {}
        torch.testing.assert_close(mine(want, pixel_values=pixels, **mine_types).logits[:, -1], ref, rtol=1e-4, atol=1e-4)


def test_llama4_with_images_matches_hugging_face(tmp_path):
    """Vision tower (class token last, interleaved 2-D rotary pairs, 2 x 2 patch folding adapter), bias-free projector and the
    Llama 4 text decoder with chunked local layers and experts; checkpoint round trip."""
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    if not hasattr(transformers, "Llama4ForConditionalGeneration"):
        pytest.skip("transformers has no Llama 4")
    torch.manual_seed(0)
    tc = dict(vocab_size=128, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=48,
              intermediate_size_mlp=96, num_hidden_layers=2, num_local_experts=4, num_experts_per_tok=1, attention_chunk_size=8,
              interleave_moe_layer_step=2, floor_scale=4, attn_scale=0.3, max_position_embeddings=128, pad_token_id=0)
    vc = dict(hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=128, image_size=16, patch_size=4, num_channels=3,
              vision_output_dim=48, projector_input_dim=48, projector_output_dim=48, pixel_shuffle_ratio=0.5)
    hf = transformers.Llama4ForConditionalGeneration(transformers.Llama4Config(
        text_config=tc, vision_config=vc, image_token_index=127, boi_token_index=125, eoi_token_index=126)).eval()
    hf.save_pretrained(str(tmp_path / "hf"))
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    assert mine.config.num_image_tokens == 4
    ids = torch.tensor([[1, 5, 125] + [127] * 4 + [126, 6, 7, 8, 9, 10], [1, 125] + [127] * 4 + [126, 16, 17, 18, 19, 20, 21]])
    pixels = torch.randn(2, 3, 16, 16)
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels).logits
        torch.testing.assert_close(mine(ids, pixel_values=pixels).logits, want, rtol=1e-4, atol=1e-4)
    labels = torch.cat([ids[:, 1:], torch.full_like(ids[:, :1], -100)], 1).masked_fill(ids.roll(-1, 1) >= 125, -100)
    mine(ids, pixel_values=pixels, labels=labels).loss.backward()
    assert mine.vision_tower.class_embedding.grad.abs().sum() > 0 and mine.projector.weight.grad.abs().sum() > 0
    mine.save_pretrained(str(tmp_path / "mine"))
    back = transformers.Llama4ForConditionalGeneration.from_pretrained(str(tmp_path / "mine")).eval()
    with torch.no_grad():
        torch.testing.assert_close(back(input_ids=ids, pixel_values=pixels).logits, want, rtol=1e-5, atol=1e-5)


def test_paddleocr_vl_matches_hugging_face(tmp_path):
    """Variable-resolution SigLIP-style tower (bilinearly resampled positions, 2-D rotary, raster-order 2 x 2 merge) and the dense
    decoder with multimodal rotary sections, two images of different sizes in one row; checkpoint round trip."""
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    if not hasattr(transformers, "PaddleOCRVLForConditionalGeneration"):
        pytest.skip("transformers has no PaddleOCR-VL")
    torch.manual_seed(0)
    hf = transformers.PaddleOCRVLForConditionalGeneration(transformers.PaddleOCRVLConfig(
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, image_size=16, patch_size=4,
                           spatial_merge_size=2),
        text_config=dict(vocab_size=300, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=16, max_position_embeddings=256,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [4, 2, 2]}),
        image_token_id=299, video_token_id=298, vision_start_token_id=297, vision_end_token_id=296)).eval()
    hf.save_pretrained(str(tmp_path / "hf"))
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    grid = torch.tensor([[1, 4, 6], [1, 2, 2]])
    pixels = torch.randn(int(grid.prod(-1).sum()), 3, 4, 4)
    ids = torch.tensor([[5, 6, 297] + [299] * 6 + [296, 7, 8, 9, 297, 299, 296, 10, 11]])
    types = (ids == 299).int()
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits
        torch.testing.assert_close(mine(ids, pixel_values=pixels, image_grid_thw=grid).logits, want, rtol=1e-4, atol=1e-4)
    labels = torch.cat([ids[:, 1:], torch.full_like(ids[:, :1], -100)], 1).masked_fill(ids.roll(-1, 1) >= 296, -100)
    mine(ids, pixel_values=pixels, image_grid_thw=grid, labels=labels).loss.backward()
    assert mine.visual.position_embedding.weight.grad.abs().sum() > 0
    mine.save_pretrained(str(tmp_path / "mine"))
    back = transformers.PaddleOCRVLForConditionalGeneration.from_pretrained(str(tmp_path / "mine")).eval()
    with torch.no_grad():
        torch.testing.assert_close(back(input_ids=ids, pixel_values=pixels, image_grid_thw=grid, mm_token_type_ids=types).logits, want,
                                   rtol=1e-5, atol=1e-5)


def test_classification_heads_match_hugging_face(tmp_path):
    """Sequence classification (last non-padding token, bias-free score) and token classification (biased score) on the unified
    decoder against transformers, checkpoint round trip, and a one-score reward head started from a causal-LM checkpoint."""
    from paddleformers_b200.transformers.auto import AutoModelForSequenceClassification, AutoModelForTokenClassification

    torch.manual_seed(0)
    kw = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, pad_token_id=0)
    ids = torch.randint(1, 128, (3, 10))
    ids[0, 7:] = 0
    ids[2, 4:] = 0
    hf = transformers.Qwen3ForSequenceClassification(transformers.Qwen3Config(num_labels=3, **kw)).eval()
    hf.save_pretrained(str(tmp_path / "seq"))
    mine = AutoModelForSequenceClassification.from_pretrained(str(tmp_path / "seq"), dtype=torch.float32).eval()
    labels = torch.tensor([0, 2, 1])
    with torch.no_grad():
        want, got = hf(input_ids=ids, labels=labels), mine(ids, labels=labels)
    assert mine.num_labels == 3 and (want.logits - got.logits).abs().max() < 1e-5 and abs(want.loss.item() - got.loss.item()) < 1e-5
    mine.save_pretrained(str(tmp_path / "seq_back"))
    back = transformers.Qwen3ForSequenceClassification.from_pretrained(str(tmp_path / "seq_back")).eval()
    with torch.no_grad():
        assert (back(input_ids=ids).logits - want.logits).abs().max() < 1e-5

    hf_tok = transformers.LlamaForTokenClassification(transformers.LlamaConfig(num_labels=5, **kw)).eval()
    hf_tok.save_pretrained(str(tmp_path / "tok"))
    tok = AutoModelForTokenClassification.from_pretrained(str(tmp_path / "tok"), dtype=torch.float32).eval()
    tags = torch.randint(0, 5, (3, 10))
    tags[0, 7:] = -100
    with torch.no_grad():
        want, got = hf_tok(input_ids=ids, labels=tags), tok(ids, labels=tags)
    assert (want.logits - got.logits).abs().max() < 1e-5 and abs(want.loss.item() - got.loss.item()) < 1e-5

    lm = transformers.LlamaForCausalLM(transformers.LlamaConfig(**kw)).eval()
    lm.save_pretrained(str(tmp_path / "lm"))
    reward = AutoModelForSequenceClassification.from_pretrained(str(tmp_path / "lm"), dtype=torch.float32, num_labels=1)
    out = reward(ids, labels=torch.tensor([0.5, -1.0, 2.0]))
    out.loss.backward()
    assert out.logits.shape == (3, 1) and reward.score.weight.grad.abs().sum() > 0
    with torch.no_grad():                            # the decoder really came from the causal-LM checkpoint
        hidden = lm.model(input_ids=ids).last_hidden_state
    assert (reward.hidden(ids) - hidden).abs().max() < 1e-4


_G4_LAYERS = ["sliding_attention", "full_attention", "sliding_attention", "sliding_attention", "full_attention", "full_attention"]


@pytest.mark.parametrize("variant", [
    dict(),                                                                                 # dense with per-layer inputs
    dict(num_kv_shared_layers=3, use_double_wide_mlp=True, layer_types=_G4_LAYERS),          # later layers reuse keys / values
    dict(attention_k_eq_v=True, num_global_key_value_heads=1, hidden_size_per_layer_input=0),
    dict(enable_moe_block=True, num_experts=8, top_k_experts=2, moe_intermediate_size=32, attention_k_eq_v=True,
         num_global_key_value_heads=1, hidden_size_per_layer_input=0),                       # the 26B-A4B layout
], ids=["dense_ple", "kv_shared_wide_mlp", "k_eq_v", "moe"])
def test_gemma4_text_matches_hugging_face(tmp_path, variant):
    """Per-layer-type head geometry, proportional rotary on the global layers, weightless value norm, unit score scale, the
    dense + routed feed-forward sum with its five norms, per-layer inputs, shared keys / values, layer scalars, capped logits:
    logits, loss and gradients against the ``transformers`` implementation; packed documents; greedy decoding; round trip."""
    from transformers import Gemma4ForCausalLM as HFModel
    from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig as HFConfig

    from paddleformers_b200.generation.utils import GenerationConfig

    torch.manual_seed(0)
    kw = dict(vocab_size=160, hidden_size=64, intermediate_size=96, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, global_head_dim=32, sliding_window=8, vocab_size_per_layer_input=160, hidden_size_per_layer_input=8,
              max_position_embeddings=128, final_logit_softcapping=30.0)
    kw.update(variant)
    cfg = HFConfig(**kw)
    cfg._attn_implementation = "eager"
    hf = HFModel(cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or "scale" in n:
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if n.endswith("layer_scalar"):
                b.copy_(torch.rand(1) + 0.5)
    hf.save_pretrained(tmp_path / "hf")
    mine = AutoModelForCausalLM.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    assert type(mine).__name__ == "Gemma4ForCausalLM"
    ids = torch.randint(3, 160, (2, 24))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = mine(ids).logits
    assert (want - got).abs().max() < 2e-4
    # loss and gradients (labels here are already next-token targets)
    labels = torch.cat([ids[:, 1:], torch.full((2, 1), -100)], dim=1)
    mine.train()
    mine(ids, labels=labels).loss.backward()
    hf_loss = hf(input_ids=ids, labels=ids).loss
    hf_loss.backward()
    assert abs(mine(ids, labels=labels).loss.item() - hf_loss.item()) < 1e-4
    ga, gb = mine.model.layers[1].self_attn.q_proj.weight.grad, hf.model.layers[1].self_attn.q_proj.weight.grad
    assert (ga - gb).abs().max() < 1e-4 * max(1.0, gb.abs().max().item())
    if variant.get("enable_moe_block"):
        ga, gb = mine.model.layers[0].moe.experts.gate_up_proj.grad, hf.model.layers[0].experts.gate_up_proj.grad
        assert (ga - gb).abs().max() < 1e-4 * max(1.0, gb.abs().max().item()) and ga.abs().sum() > 0
        assert mine.model.layers[0].moe.router.per_expert_scale.grad.abs().sum() > 0
    mine.eval()
    # two packed documents: the second one's logits equal those of the document alone (positions restart)
    kend = torch.full((2, 24), 24, dtype=torch.int32)
    kend[:, :10] = 10
    pos = torch.cat([torch.arange(10), torch.arange(14)])[None].expand(2, -1)
    with torch.no_grad():
        packed = mine(ids, position_ids=pos, kend=kend).logits
        alone = mine(ids[:, 10:]).logits
    assert (packed[:, 10:] - alone).abs().max() < 2e-4
    # greedy decoding agrees with the argmax of a full forward
    out = mine.generate(ids[:, :9], GenerationConfig(max_new_tokens=4, eos_token_id=-1))
    with torch.no_grad():
        step = hf(input_ids=out[:, :-1]).logits.argmax(-1)
    assert out.shape == (2, 13) and torch.equal(step[:, 8:], out[:, 9:])
    mine.save_pretrained(str(tmp_path / "mine"))
    back = HFModel.from_pretrained(tmp_path / "mine").eval()
    with torch.no_grad():
        assert (back(input_ids=ids).logits - want).abs().max() < 1e-5


def test_gemma4_reads_the_multimodal_wrapper_configuration_and_the_reference_field_names():
    from paddleformers_b200.transformers.auto import AutoConfig

    cfg = AutoConfig.for_model("gemma4", num_hidden_layers=12, interleaved_attn_pattern=(5, 1), full_attention_rope_base=5e5,
                               hidden_act="gelu_pytorch_tanh", enable_moe_block=True, num_experts=8, top_k_experts=2)
    assert cfg.model_type == "gemma4_text" and cfg.layer_types[5] == "full_attention" and cfg.layer_types[-1] == "full_attention"
    assert cfg.rope_parameters["full_attention"] == {"rope_type": "proportional", "rope_theta": 5e5, "partial_rotary_factor": 0.25}
    wrapped = type(cfg).from_dict({"model_type": "gemma4", "text_config": {"model_type": "gemma4_text", "num_hidden_layers": 3}})
    assert wrapped.num_hidden_layers == 3 and wrapped.num_experts_per_tok is None
    assert cfg.layer_head_geometry(0) == (256, 4, False) and cfg.layer_head_geometry(5)[0] == 512


def test_ernie4_5_vl_matches_hugging_face(tmp_path):
    """Vision tower, spatial + temporal resampler (a still image paired with itself, video frames paired even / odd), three-axis
    rotary positions on interleaved pairs, text / vision expert groups with their own routers and widths, shared experts:
    logits for an image prompt, an image + video prompt and plain text; loss and gradients; the published checkpoint layout
    (experts numbered text first, transposed routers, two-row correction bias) both ways."""
    from transformers.models.ernie4_5_vl_moe.configuration_ernie4_5_vl_moe import Ernie4_5_VLMoeConfig as HFConfig
    from transformers.models.ernie4_5_vl_moe.modeling_ernie4_5_vl_moe import Ernie4_5_VLMoeForConditionalGeneration as HFModel

    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(0)
    cfg = HFConfig(
        text_config=dict(vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4,
                         num_key_value_heads=2, moe_intermediate_size=[32, 16], moe_k=2, moe_num_experts=4, moe_num_shared_experts=1,
                         max_position_embeddings=256, mlp_layer_types=["dense", "sparse", "sparse"], router_aux_loss_coef=0.0,
                         rope_parameters={"rope_theta": 10000.0, "rope_type": "default", "mrope_section": [3, 3, 2]}),
        vision_config=dict(depth=2, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=4, spatial_merge_size=2,
                           temporal_merge_size=2),
        image_token_id=190, video_token_id=191, image_start_token_id=192, image_end_token_id=193, video_start_token_id=194,
        video_end_token_id=195)
    cfg._attn_implementation = "eager"
    hf = HFModel(cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "e_score_correction_bias" in n:
                p.copy_(torch.randn_like(p) * 0.1)
            if "norm" in n or ".ln." in n:
                p.add_(torch.randn_like(p) * 0.1)
    hf.save_pretrained(tmp_path / "hf")
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    # an image of 4 x 6 patches (6 tokens after the 2 x 2 merge), then a video of 4 frames of 4 x 4 patches (2 frame pairs x 4)
    ids = [5, 6, 192] + [190] * 6 + [193, 7, 8, 9]
    mm = [0, 0, 0] + [1] * 6 + [0, 0, 0, 0]
    moe = [0, 0, 1] + [1] * 6 + [1, 0, 0, 0]
    img = dict(pixel_values=torch.randn(24, 48), image_grid_thw=torch.tensor([[1, 4, 6]]))
    vid = dict(pixel_values_videos=torch.randn(64, 48), video_grid_thw=torch.tensor([[4, 4, 4]]))
    ids2 = ids + [194] + [191] * 8 + [195, 10, 11]
    mm2, moe2 = mm + [0] + [2] * 8 + [0, 0, 0], moe + [2] + [2] * 8 + [2, 0, 0]
    t = lambda x: torch.tensor([x])          # noqa: E731
    with torch.no_grad():
        assert (hf(input_ids=t(ids), mm_token_type_ids=t(mm), moe_mm_token_type_ids=t(moe), **img).logits
                - mine(t(ids), **img).logits).abs().max() < 1e-4
        want = hf(input_ids=t(ids2), mm_token_type_ids=t(mm2), moe_mm_token_type_ids=t(moe2), **img, **vid).logits
        assert (want - mine(t(ids2), **img, **vid).logits).abs().max() < 1e-4
        text = torch.randint(0, 180, (2, 12))
        assert (hf(input_ids=text).logits - mine(text).logits).abs().max() < 1e-4
    pos = mine.forward.__globals__["multimodal_position_ids"](t(ids2), 190, 191, img["image_grid_thw"], torch.tensor([[2, 4, 4]]), 2)
    assert pos[:, 0, 3:9].tolist() == [[3] * 6, [3, 3, 3, 4, 4, 4], [3, 4, 5] * 2]           # t fixed, rows, columns
    assert pos[0, 0, 9].item() == 6 and pos[:, 0, 14:22].tolist()[0] == [11] * 8             # text resumes after max(rows, cols)
    # loss and gradients; labels are next-token targets here, shifted inside the other implementation
    lab = torch.tensor(ids2[1:] + [-100])[None]
    lab[lab >= 190] = -100
    hf_lab = torch.tensor(ids2)[None].clone()
    hf_lab[hf_lab >= 190] = -100
    mine.train()
    out = mine(t(ids2), labels=lab, **img, **vid)
    out.loss.backward()
    ref = hf(input_ids=t(ids2), labels=hf_lab, mm_token_type_ids=t(mm2), moe_mm_token_type_ids=t(moe2), **img, **vid)
    ref.loss.backward()
    assert abs(out.loss.item() - ref.loss.item()) < 1e-4
    ga = mine.language.model.layers["1"].mlp.vision_moe.experts.down_proj.grad
    gb = hf.model.language_model.layers[1].mlp.vision_moe.experts.down_proj.grad
    assert ga.abs().sum() > 0 and (ga - gb).abs().max() < 1e-4 * max(1.0, gb.abs().max().item())
    ga, gb = mine.resampler.temporal_linear.fc1.weight.grad, hf.model.resampler_model.temporal_linear.fc1.weight.grad
    assert (ga - gb).abs().max() < 1e-4 * max(1.0, gb.abs().max().item())
    mine.eval()
    mine.save_pretrained(str(tmp_path / "mine"))
    back = HFModel.from_pretrained(tmp_path / "mine").eval()
    with torch.no_grad():
        again = back(input_ids=t(ids2), mm_token_type_ids=t(mm2), moe_mm_token_type_ids=t(moe2), **img, **vid).logits
    assert (again - want).abs().max() < 1e-5


def test_ernie4_5_vl_trains_on_a_padded_batch_of_images_of_different_sizes():
    """The VL data path (single-frame patches in merge-block order, one placeholder per merged patch, padded batch) through the
    model and an optimizer step; vision rows are found from the token ids."""
    import numpy as np

    from paddleformers_b200.models.ernie4_5_vl import Ernie4_5VLConfig, Ernie4_5VLForConditionalGeneration
    from paddleformers_b200.models.vision_language import mm_collate_fn
    from paddleformers_b200.transformers.image_processing import Qwen2VLImageProcessor

    torch.manual_seed(0)
    cfg = Ernie4_5VLConfig(
        text_config=dict(vocab_size=200, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, moe_intermediate_size=[32, 16], moe_k=2, moe_num_experts=4, moe_num_shared_experts=1,
                         mlp_layer_types=["dense", "sparse"], rope_parameters={"rope_theta": 10000.0, "mrope_section": [3, 3, 2]}),
        vision_config=dict(depth=1, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=4, spatial_merge_size=2),
        image_token_id=190, video_token_id=191, image_start_token_id=192, image_end_token_id=193, video_start_token_id=194,
        video_end_token_id=195)
    assert cfg.vision_start_token_id == 192 and cfg.text_config.moe_layers == [1]
    model = Ernie4_5VLForConditionalGeneration(cfg, dtype=torch.float32)
    proc = Qwen2VLImageProcessor(patch_size=4, merge_size=2, temporal_patch_size=1, min_pixels=64, max_pixels=1024)
    rng = np.random.default_rng(0)
    examples = []
    for hw in ((16, 24), (32, 16)):
        pre = proc([rng.integers(0, 255, (*hw, 3), dtype=np.uint8)])
        n = proc.num_image_tokens(pre["image_grid_thw"][0].tolist())
        ids = [5, 192] + [190] * n + [193] + rng.integers(1, 180, 6).tolist()
        lab = [-100] * (n + 2) + ids[n + 3:] + [-100]
        examples.append({"input_ids": torch.tensor(ids), "labels": torch.tensor(lab), **pre})
    batch = mm_collate_fn(examples, pad_token_id=0)
    assert batch["input_ids"].shape[0] == 2 and batch["pixel_values"].shape[1] == 3 * 4 * 4
    rows = model.vision_rows(batch["input_ids"])
    assert rows.sum().item() == sum(int((e["input_ids"] >= 190).sum()) for e in examples)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    losses = []
    for _ in range(4):
        out = model(**batch)
        out.loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(out.loss.item())
    assert losses[-1] < losses[0]
    assert all(m.mlp.vision_rows is None for m in model.language.model.layers.values() if hasattr(m.mlp, "vision_rows"))


def test_phi4_multimodal_matches_hugging_face(tmp_path):
    """Image branch (fractional position buckets, partly filled crops, 2 x 2 pooling, row / image separators), audio branch
    (convolutional time reduction, conformer blocks with relative-position bias, windows of 500 frames for long audio, the two
    projector sets), placeholders replaced in the prompt, Phi-3 decoder: logits, loss and gradients; checkpoint both ways.
    Padded audio frames must not influence the valid ones."""
    from transformers.models.phi4_multimodal.configuration_phi4_multimodal import Phi4MultimodalConfig as HFConfig
    from transformers.models.phi4_multimodal.modeling_phi4_multimodal import Phi4MultimodalForCausalLM as HFModel

    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    torch.manual_seed(0)
    cfg = HFConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, max_position_embeddings=2048, original_max_position_embeddings=2048, pad_token_id=0,
                   bos_token_id=1, eos_token_id=2,
                   vision_config=dict(hidden_size=32, intermediate_size=48, num_hidden_layers=3, num_attention_heads=2, image_size=56,
                                      patch_size=14, crop_size=56, image_token_id=290),
                   audio_config=dict(hidden_size=32, intermediate_size=48, num_blocks=2, num_attention_heads=2, ext_pw_out_channel=32,
                                     depthwise_separable_out_channel=32, input_size=16, nemo_conv_channels=8, nemo_final_size=2,
                                     time_reduction=8, bias_max_distance=20, audio_token_id=291))
    for c in (cfg, cfg.vision_config, cfg.audio_config):
        c._attn_implementation = "eager"
    hf = HFModel(cfg).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "extensor" in n or n.endswith((".b1", ".b2")) or "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if "global_mean" in n:
                b.copy_(torch.randn_like(b) * 0.1)
            if "global_invstd" in n:
                b.copy_(torch.rand_like(b) + 0.5)
    hf.save_pretrained(tmp_path / "hf")
    mine = AutoModelForConditionalGeneration.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    # image resized to 56 x 112: global view + 1 x 2 crops of 4 x 4 patches; the right crop shows the image in its two left
    # patch columns only
    pix = torch.randn(1, 3, 3, 56, 56)
    sizes = torch.tensor([[56, 112]])
    mask = torch.ones(1, 3, 4, 4)
    mask[0, 2, :, 2:] = 0
    n_img = 2 * (3 + 1) + 1 + 2 * (2 + 1)            # tiled crops: 2 rows of 3 useful columns + separator; separator; global 2 x (2 + 1)
    feats = torch.randn(1, 40, 16)
    n_aud = 5                                         # 40 frames / 8
    ids = torch.tensor([[5, 6] + [290] * n_img + [7] + [291] * n_aud + [8, 9]])
    kw = dict(image_pixel_values=pix, image_sizes=sizes, image_attention_mask=mask, audio_input_features=feats,
              audio_embed_sizes=torch.tensor([n_aud]))
    with torch.no_grad():
        want = hf(input_ids=ids, **kw).logits
        assert (want - mine(ids, **kw).logits).abs().max() < 1e-4
        # audio only ("speech" projectors), longer than one window of 500 reduced frames
        long = torch.randn(1, 8 * 520, 16)
        ids2 = torch.tensor([[5] + [291] * 520 + [8, 9]])
        a = hf(input_ids=ids2, audio_input_features=long, audio_embed_sizes=torch.tensor([520])).logits
        b = mine(ids2, audio_input_features=long, audio_embed_sizes=torch.tensor([520])).logits
        assert (a - b).abs().max() < 1e-4
        # padding: frames beyond the valid length change nothing in the valid part
        enc = mine.embed_tokens_extend.audio_embed.encoder
        x = torch.randn(1, 64, 16)
        fm = torch.zeros(1, 64, dtype=torch.bool)
        fm[:, :40] = True
        y1 = enc(x, fm)
        x2 = x.clone()
        x2[:, 48:] = 7.0                               # past the receptive field of the last valid reduced frame
        y2 = enc(x2, fm)
        assert (y1[:, :5] - y2[:, :5]).abs().max() < 1e-5 and (y1[:, 6:] - y2[:, 6:]).abs().max() > 1e-6
    lab = torch.cat([ids[:, 1:], torch.full((1, 1), -100)], dim=1)
    lab[lab >= 290] = -100
    hf_lab = ids.clone()
    hf_lab[hf_lab >= 290] = -100
    mine.train()
    out = mine(ids, labels=lab, **kw)
    out.loss.backward()
    ref = hf(input_ids=ids, labels=hf_lab, **kw)
    ref.loss.backward()
    assert abs(out.loss.item() - ref.loss.item()) < 1e-4
    pairs = [(mine.embed_tokens_extend.image_embed.sub_img_feature_extensor, hf.model.embed_tokens_extend.image_embed.sub_img_feature_extensor),
             (mine.embed_tokens_extend.audio_embed.encoder.encoders[0].conv.b1, hf.model.embed_tokens_extend.audio_embed.encoder.encoders[0].conv.glu.b1),
             (mine.embed_tokens_extend.image_embed.img_processor.position_embedding.weight,
              hf.model.embed_tokens_extend.image_embed.img_processor.embeddings.position_embedding.weight)]
    for a, b in pairs:
        assert a.grad.abs().sum() > 0 and (a.grad - b.grad).abs().max() < 1e-4 * max(1.0, b.grad.abs().max().item())
    mine.eval()
    mine.save_pretrained(str(tmp_path / "mine"))
    back = HFModel.from_pretrained(tmp_path / "mine").eval()
    with torch.no_grad():
        assert (back(input_ids=ids, **kw).logits - want).abs().max() < 1e-5


def test_molmo_decoder_and_tower_against_olmo2_and_clip_oracles(tmp_path):
    """No other implementation of Molmo is at hand, so its parts are checked against the models they are built from: the
    decoder (norms after the branches, full-width QK norm, fused [q | k | v] and [up | gate] projections, extended embedding
    table, head over the base table) against ``transformers``' OLMo 2 through a checkpoint written in Molmo's tensor names; the
    image tower against ``transformers``' CLIP vision encoder; pooling, padding embeddings and the scatter-add into the token
    embeddings against a direct restatement."""
    from safetensors.torch import save_file
    from transformers import CLIPVisionConfig, CLIPVisionModel, Olmo2Config, Olmo2ForCausalLM

    from paddleformers_b200.models.molmo import MolmoConfig, MolmoForCausalLM

    torch.manual_seed(0)
    E, A, H, I, L = 96, 8, 64, 80, 2
    hf = Olmo2ForCausalLM(Olmo2Config(vocab_size=E, hidden_size=H, intermediate_size=I, num_hidden_layers=L, num_attention_heads=4,
                                      num_key_value_heads=2, max_position_embeddings=128, rope_theta=10000.0, rms_norm_eps=1e-6,
                                      tie_word_embeddings=False, pad_token_id=0)).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    clip = CLIPVisionModel(CLIPVisionConfig(hidden_size=32, intermediate_size=48, num_hidden_layers=4, num_attention_heads=2,
                                            image_size=28, patch_size=14, hidden_act="quick_gelu", layer_norm_eps=1e-5)).eval()
    sd, T, V = {}, "model.transformer.", "model.vision_backbone."
    hs = hf.state_dict()
    sd[T + "wte.embedding"] = hs["model.embed_tokens.weight"]
    sd[T + "wte.new_embedding"] = torch.randn(A, H) * 0.02
    sd[T + "ln_f.weight"] = hs["model.norm.weight"]
    sd[T + "ff_out.weight"] = hs["lm_head.weight"]
    for i in range(L):
        a, b = f"model.layers.{i}.", f"{T}blocks.{i}."
        sd[b + "att_proj.weight"] = torch.cat([hs[a + f"self_attn.{x}_proj.weight"] for x in "qkv"], dim=0)
        sd[b + "attn_out.weight"] = hs[a + "self_attn.o_proj.weight"]
        sd[b + "ff_proj.weight"] = torch.cat([hs[a + "mlp.up_proj.weight"], hs[a + "mlp.gate_proj.weight"]], dim=0)
        sd[b + "ff_out.weight"] = hs[a + "mlp.down_proj.weight"]
        sd[b + "attn_norm.weight"] = hs[a + "post_attention_layernorm.weight"]
        sd[b + "ff_norm.weight"] = hs[a + "post_feedforward_layernorm.weight"]
        sd[b + "q_norm.weight"], sd[b + "k_norm.weight"] = hs[a + "self_attn.q_norm.weight"], hs[a + "self_attn.k_norm.weight"]
    cs = clip.state_dict()
    pre = "vision_model."
    sd[V + "image_vit.class_embedding"] = cs[pre + "embeddings.class_embedding"]
    sd[V + "image_vit.positional_embedding"] = cs[pre + "embeddings.position_embedding.weight"]
    sd[V + "image_vit.patch_embedding.weight"] = cs[pre + "embeddings.patch_embedding.weight"].permute(0, 2, 3, 1).reshape(32, -1)
    sd[V + "image_vit.pre_ln.weight"], sd[V + "image_vit.pre_ln.bias"] = cs[pre + "pre_layrnorm.weight"], cs[pre + "pre_layrnorm.bias"]
    for i in range(4):
        a, b = f"{pre}encoder.layers.{i}.", f"{V}image_vit.transformer.resblocks.{i}."
        for mine, theirs in (("attention.wq", "self_attn.q_proj"), ("attention.wk", "self_attn.k_proj"), ("attention.wv", "self_attn.v_proj"),
                             ("attention.wo", "self_attn.out_proj"), ("feed_forward.w1", "mlp.fc1"), ("feed_forward.w2", "mlp.fc2"),
                             ("attention_norm", "layer_norm1"), ("ffn_norm", "layer_norm2")):
            for leaf in ("weight", "bias"):
                sd[b + f"{mine}.{leaf}"] = cs[a + f"{theirs}.{leaf}"]
    cfg = MolmoConfig(vocab_size=E - 6, embedding_size=E, hidden_size=H, intermediate_size=2 * I, num_hidden_layers=L, num_attention_heads=4,
                      num_key_value_heads=2, additional_vocab_size=A, max_position_embeddings=128, rope_theta=10000.0, layer_norm_eps=1e-6,
                      vision_backbone=dict(image_default_input_size=(28, 28), image_patch_size=14, image_emb_dim=32, image_num_heads=2,
                                           image_num_key_value_heads=2, image_num_layers=4, image_head_dim=16, image_mlp_dim=48,
                                           image_num_pos=5, image_norm_eps=1e-5), vit_layers=(-1, -3))
    mine = MolmoForCausalLM(cfg, dtype=torch.float32)
    for n, p in mine.model.vision_backbone.named_parameters():            # pooling, projector, padding embeddings: random
        if ("model.vision_backbone." + n) not in sd:
            sd["model.vision_backbone." + n] = torch.randn_like(p) * 0.1
    ck = tmp_path / "molmo"
    ck.mkdir()
    save_file({k: v.contiguous() for k, v in sd.items()}, str(ck / "model.safetensors"))
    cfg.save_pretrained(str(ck))
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    mine = AutoModelForConditionalGeneration.from_pretrained(str(ck), dtype=torch.float32).eval()
    assert type(mine).__name__ == "MolmoForCausalLM"
    ids = torch.randint(0, E, (2, 14))
    with torch.no_grad():
        assert (hf(input_ids=ids).logits - mine(ids).logits).abs().max() < 1e-4          # decoder, text only
        extra = mine(torch.tensor([[E + 3, 5, 6]])).logits                                # a row of the extra table is reachable
        assert extra.shape == (1, 3, E)
        # tower: every block's output equals the CLIP encoder's hidden states
        img = torch.randn(3, 3, 28, 28)
        patches = img.reshape(3, 3, 2, 14, 2, 14).permute(0, 2, 4, 3, 5, 1).reshape(3, 4, 14 * 14 * 3)
        outs = mine.model.vision_backbone.image_vit(patches, (2, 2))
        want = clip(pixel_values=img, output_hidden_states=True).hidden_states
        for i in range(4):
            assert (outs[i] - want[i + 1]).abs().max() < 1e-4
        # backbone after the tower, restated directly
        vb = mine.model.vision_backbone
        images = patches.reshape(1, 3, 4, -1).clone()
        images[0, 2] = -1                                                                 # an unused crop
        masks = torch.ones(1, 3, 4)
        masks[0, 1, 2:] = 0.0
        masks[0, 1, 1] = 0.25
        got = vb(images, masks)
        feats = torch.cat([outs[-1], outs[-3]], dim=-1)[:, 1:].clone()
        feats[2] = 0
        feats = feats + vb.pad_embed[0] * (masks[0] == 0)[..., None] + vb.pad_embed[1] * ((masks[0] < 1) & (masks[0] > 0))[..., None]
        rows = []
        for c in range(3):
            blk = feats[c]                                                                # 2 x 2 patches = one pooled row
            q = blk.mean(0, keepdim=True)
            pa = vb.image_pooling_2d
            qh = pa.wq(q).view(1, 2, 16).transpose(0, 1)
            kh, vh = pa.wk(blk).view(4, 2, 16).transpose(0, 1), pa.wv(blk).view(4, 2, 16).transpose(0, 1)
            att = torch.softmax(qh @ kh.transpose(1, 2) / 4.0, dim=-1) @ vh
            o = pa.wo(att.transpose(0, 1).reshape(1, 32))
            pr = vb.image_projector
            rows.append(pr["w2"](torch.nn.functional.silu(pr["w1"](o)) * pr["w3"](o)))
        assert (got[0, :, 0] - torch.cat(rows)).abs().max() < 1e-5
        # the rows are added at image_input_idx; -1 rows are ignored
        idx = torch.tensor([[[3], [7], [-1]]])
        base = mine.language.model.embed(ids[:1]).clone()
        with_img = mine(ids[:1], images=images, image_masks=masks, image_input_idx=idx).logits
        h = base.clone()
        h[3] += got[0, 0, 0]
        h[7] += got[0, 1, 0]
        lm = mine.language
        ctx = lm.model.make_context(ids[:1])
        hid, res = lm.model.run_layers(h, None, ctx)
        hid = lm.model.norm(hid, res)[0] if res is not None else lm.model.norm(hid)
        assert (with_img[0] - torch.nn.functional.linear(hid, mine.head_weight())).abs().max() < 1e-5
    mine.train()
    out = mine(ids[:1], images=images, image_masks=masks, image_input_idx=idx, labels=ids[:1])
    out.loss.backward()
    assert mine.model.vision_backbone.pad_embed.grad.abs().sum() > 0 and mine.lm_head.weight.grad.abs().sum() > 0
    mine.save_pretrained(str(tmp_path / "again"))
    from safetensors import safe_open

    with safe_open(str(tmp_path / "again" / "model.safetensors"), "pt") as f:
        assert set(f.keys()) == set(sd) and torch.equal(f.get_tensor(T + "blocks.1.ff_proj.weight"), sd[T + "blocks.1.ff_proj.weight"])
        assert f.get_tensor(T + "wte.new_embedding").shape == (A, H)
