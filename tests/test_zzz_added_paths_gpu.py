"""GPU checks of paths that go through the existing kernels with new inputs, or around them in tensor operations:
sliding-window / chunk bounds on the flash attention kernels, the optimizer variants and sharding stage 3 on flat device
buffers, the linear-attention mixers and the eager attention variants on the device. Every comparison is against an fp32
PyTorch computation of the same quantity. The file name sorts last so that a run that stops at the first failure has already
executed every kernel test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(scope="module")
def F():
    from paddleformers_b200.ops import functional as F

    return F


@pytest.mark.parametrize("kind,width", [("window", 96), ("window", 300), ("chunk", 128), ("chunk", 200)])
def test_window_and_chunk_bounds_on_the_flash_kernels(F, kind, width):
    """Sliding windows and attention chunks are per-key "first masked row" bounds, the same input as packed-document masks:
    forward and backward against the fp32 reference with the same bound."""
    torch.manual_seed(0)
    B, S, Hq, Hkv = 2, 640, 4, 2
    j = torch.arange(S, dtype=torch.int32)
    bound = (j + width) if kind == "window" else ((j // width + 1) * width)
    kend = bound.clamp(max=S)[None].expand(B, S).contiguous().cuda()
    q = torch.randn(B, S, Hq, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, S, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = F.flash_attention(q, k, v, causal=True, kend=kend)
    g = torch.randn_like(out)
    out.backward(g)
    F.check_kernel_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = F.attention_reference(qr, kr, vr, causal=True, kend=kend)
    ref.backward(g.float())
    assert _rel_err(out, ref) < 2e-2
    assert _rel_err(q.grad, qr.grad) < 3e-2 and _rel_err(k.grad, kr.grad) < 3e-2 and _rel_err(v.grad, vr.grad) < 3e-2
    # the bound really hides keys: the last row must differ from plain causal attention
    plain = F.flash_attention(q.detach(), k.detach(), v.detach(), causal=True)
    assert _rel_err(out[:, -1], plain[:, -1]) > 1e-2


def _tiny(dtype, device, **over):
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.transformers.auto import AutoModelForCausalLM

    cfg = named_config("llama3-8b", num_hidden_layers=2, hidden_size=512, intermediate_size=1408, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=128, vocab_size=4096, **over)
    torch.manual_seed(0)
    return AutoModelForCausalLM.from_config(cfg, dtype=dtype, device=device), cfg


def _steps(model, opt, n=3, seed=1):
    g = torch.Generator().manual_seed(seed)
    losses = []
    for _ in range(n):
        ids = torch.randint(0, 4096, (2, 256), generator=g).cuda()
        out = model(ids, labels=torch.roll(ids, -1, 1))
        out.loss.backward()
        opt.accumulate_grads()
        opt.step()
        losses.append(float(out.loss))
    return losses


def test_mistral_style_window_model_matches_its_fp32_path(F):
    from paddleformers_b200.models.configuration import MistralConfig
    from paddleformers_b200.transformers.auto import AutoModelForCausalLM

    kw = dict(num_hidden_layers=2, hidden_size=512, intermediate_size=1408, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
              vocab_size=4096, sliding_window=64)
    torch.manual_seed(0)
    ref = AutoModelForCausalLM.from_config(MistralConfig(**kw), dtype=torch.float32)
    gpu = AutoModelForCausalLM.from_config(MistralConfig(**kw), dtype=torch.bfloat16, device="cuda")
    sd = {k: v.to(torch.bfloat16) for k, v in ref.state_dict().items()}
    gpu.load_state_dict(sd)
    ref.load_state_dict({k: v.float() for k, v in sd.items()})
    ids = torch.randint(0, 4096, (2, 256))
    a, b = ref(ids, labels=ids), gpu(ids.cuda(), labels=ids.cuda())
    F.check_kernel_status()
    assert abs(a.loss.item() - b.loss.item()) / a.loss.item() < 0.03


def test_optimizer_variants_follow_the_fused_kernel_on_device_shards():
    """bf16 moments, host-resident moments and the one-second-moment-per-row rule run as tensor operations on the same flat
    device buffers the fused AdamW kernel uses; with fp32 moments the trajectory must coincide with the kernel's."""
    from paddleformers_b200.parallel.sharding import ShardedAdamW
    from paddleformers_b200.utils.optimizer import AdamWCustom, AdamWMini

    kw = dict(lr=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    base_model, _ = _tiny(torch.bfloat16, "cuda")
    base = _steps(base_model, ShardedAdamW(base_model, **kw))
    for make in (lambda m: AdamWCustom(m, **kw), lambda m: AdamWCustom(m, offload_moments=True, offload_chunk_numel=1 << 20, **kw),
                 lambda m: AdamWCustom(m, moment_dtype=torch.bfloat16, **kw)):
        model, _ = _tiny(torch.bfloat16, "cuda")
        got = _steps(model, make(model))
        assert all(abs(a - b) / a < 2e-2 for a, b in zip(base, got)), (base, got)
    model, _ = _tiny(torch.bfloat16, "cuda")
    mini = _steps(model, AdamWMini(model, **kw), n=4)
    assert all(l == l for l in mini) and mini[-1] < mini[0] + 0.5


def test_sharding_stage3_units_run_the_kernels_through_the_shared_buffer(F):
    """One process: per-layer units (parameters as views of one shared bf16 buffer, fp32 gradient views for the weight-gradient
    kernels, recompute in backward) against the flat stage-1 optimizer on the same data."""
    from paddleformers_b200.parallel.fsdp import FullyShardedOptimizer
    from paddleformers_b200.parallel.sharding import ShardedAdamW

    kw = dict(lr=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    a_model, _ = _tiny(torch.bfloat16, "cuda")
    a = _steps(a_model, ShardedAdamW(a_model, **kw))
    b_model, _ = _tiny(torch.bfloat16, "cuda")
    opt = FullyShardedOptimizer(b_model, **kw)
    b = _steps(b_model, opt)
    F.check_kernel_status()
    assert all(abs(x - y) / x < 2e-2 for x, y in zip(a, b)), (a, b)
    ref = dict(a_model.named_parameters())
    name, p = next((n, p) for n, p in b_model.named_parameters() if n.endswith("layers.1.mlp.down_proj.weight"))
    assert _rel_err(opt.full_tensor(p), ref[name].detach().cpu()) < 2e-2


def test_linear_attention_mixers_on_the_device():
    from paddleformers_b200.nn.linear_attention import decayed_linear_attention, gated_delta_rule

    torch.manual_seed(0)
    B, S, H, dk, dv = 2, 300, 4, 32, 32
    q = torch.nn.functional.normalize(torch.randn(B, S, H, dk), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(B, S, H, dk), dim=-1)
    v, g, beta = torch.randn(B, S, H, dv), -torch.rand(B, S, H) * 0.3, torch.rand(B, S, H)
    ref, _ = gated_delta_rule(q, k, v, g, beta)
    out, _ = gated_delta_rule(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda())
    assert _rel_err(out.cpu(), ref) < 1e-3
    slope = torch.tensor([0.3, 0.1, 0.03, 0.01])
    ref2, _ = decayed_linear_attention(q, k, v, slope)
    out2, _ = decayed_linear_attention(q.cuda(), k.cuda(), v.cuda(), slope.cuda())
    assert _rel_err(out2.cpu(), ref2) < 1e-3


@pytest.mark.parametrize("family,extra", [
    ("gemma2", dict(sliding_window=64, attn_logit_softcapping=50.0, final_logit_softcapping=30.0, query_pre_attn_scalar=128)),
    ("gpt_oss", dict(sliding_window=64, num_local_experts=8, num_experts_per_tok=2, intermediate_size=256)),
    ("qwen3_next", dict(linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=64, linear_value_head_dim=64,
                        partial_rotary_factor=0.5, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256, shared_expert_intermediate_size=256)),
])
def test_families_on_tensor_operation_paths_train_in_bf16_on_the_device(F, family, extra):
    """Families whose attention variants bypass the flash kernels (soft cap, sinks, linear attention): the bf16 device run
    stays close to the fp32 host run of the same weights."""
    from paddleformers_b200.transformers.auto import AutoConfig, AutoModelForCausalLM

    kw = dict(num_hidden_layers=4 if family == "qwen3_next" else 2, hidden_size=512, intermediate_size=1024, num_attention_heads=4,
              num_key_value_heads=2, head_dim=128, vocab_size=4096)
    kw.update(extra)
    torch.manual_seed(0)
    ref = AutoModelForCausalLM.from_config(AutoConfig.for_model(family, **kw), dtype=torch.float32)
    gpu = AutoModelForCausalLM.from_config(AutoConfig.for_model(family, **kw), dtype=torch.bfloat16, device="cuda")
    sd = {k: (v.to(torch.bfloat16) if v.dtype == torch.float32 and not (k.endswith("gate.weight") or k.endswith("gate.bias")) else v)
          for k, v in ref.state_dict().items()}
    gpu.load_state_dict(sd)
    ref.load_state_dict({k: v.float() for k, v in sd.items()})
    ids = torch.randint(0, 4096, (2, 128))
    a, b = ref(ids, labels=ids), gpu(ids.cuda(), labels=ids.cuda())
    a.loss.backward()
    b.loss.backward()
    F.check_kernel_status()
    assert abs(a.loss.item() - b.loss.item()) / a.loss.item() < 0.05
    emb_r, emb_g = ref.model.embed_tokens.weight.grad, gpu.model.embed_tokens.weight
    g = getattr(emb_g, "main_grad", None)
    g = g if g is not None and g.abs().sum() > 0 else emb_g.grad
    assert g is not None and torch.isfinite(g.float()).all()


def test_paligemma_two_way_prefix_on_the_device(F):
    """SigLIP tower (head size 64: the generic attention path), projector and a Gemma decoder under the two-way prefix mask: the bf16
    device run stays close to the fp32 host run of the same weights, and gradients reach the tower."""
    from paddleformers_b200.models.paligemma import PaliGemmaConfig
    from paddleformers_b200.transformers.auto import AutoModelForConditionalGeneration

    def config():
        return PaliGemmaConfig(
            vision_config=dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2, image_size=64, patch_size=16),
            text_config=dict(model_type="gemma", hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                             num_key_value_heads=1, head_dim=128, vocab_size=4096),
            image_token_index=4095, projection_dim=512)

    torch.manual_seed(0)
    ref = AutoModelForConditionalGeneration.from_config(config(), dtype=torch.float32)
    gpu = AutoModelForConditionalGeneration.from_config(config(), dtype=torch.bfloat16, device="cuda")
    sd = {k: v.to(torch.bfloat16) for k, v in ref.state_dict().items()}
    gpu.load_state_dict(sd)
    ref.load_state_dict({k: v.float() for k, v in sd.items()})
    n_img = ref.config.num_image_tokens
    ids = torch.cat([torch.full((2, n_img), 4095), torch.randint(0, 4000, (2, 48))], dim=1)
    types = torch.cat([torch.zeros(2, n_img + 16, dtype=torch.long), torch.ones(2, 32, dtype=torch.long)], dim=1)
    labels = torch.where(types == 1, ids, torch.full_like(ids, -100)).roll(-1, 1)
    labels[:, -1] = -100
    pixels = torch.randn(2, 3, 64, 64)
    a = ref(ids, pixel_values=pixels, token_type_ids=types, labels=labels)
    b = gpu(ids.cuda(), pixel_values=pixels.cuda().to(torch.bfloat16), token_type_ids=types.cuda(), labels=labels.cuda())
    b.loss.backward()
    F.check_kernel_status()
    assert abs(a.loss.item() - b.loss.item()) / a.loss.item() < 0.05
    g = gpu.vision_tower.patch_embedding.weight.grad
    assert g is not None and torch.isfinite(g.float()).all() and g.abs().sum() > 0
