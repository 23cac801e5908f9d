"""The fused routing kernels (scores, top-k, combine weights, counts, stable ranks, balance loss) against the same router
evaluated with tensor operations, forward and backward."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _router(kind, device):
    from paddleformers_b200.models.configuration import DeepseekV3Config, Qwen3MoeConfig
    from paddleformers_b200.nn.moe import TopkRouter

    if kind == "qwen3":
        cfg = Qwen3MoeConfig(hidden_size=256, num_experts=128, num_experts_per_tok=8, moe_intermediate_size=64, intermediate_size=64,
                             num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2, vocab_size=64, router_aux_loss_coef=1e-2)
    elif kind == "dsv3":
        cfg = DeepseekV3Config(hidden_size=256, n_routed_experts=256, num_experts_per_tok=8, n_group=8, topk_group=4,
                               moe_intermediate_size=64, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                               num_key_value_heads=4, vocab_size=64, routed_scaling_factor=2.5)
    else:  # glm-like: sigmoid scores, bias-corrected selection, one group, balance loss on
        cfg = DeepseekV3Config(hidden_size=256, n_routed_experts=128, num_experts_per_tok=8, n_group=1, topk_group=1,
                               moe_intermediate_size=64, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                               num_key_value_heads=4, vocab_size=64, routed_scaling_factor=1.0, router_aux_loss_coef=1e-2)
    r = TopkRouter(cfg, dtype=torch.bfloat16, device=device)
    torch.nn.init.normal_(r.weight, std=0.5)
    if r.e_score_correction_bias is not None:
        r.e_score_correction_bias.copy_(0.05 * torch.randn_like(r.e_score_correction_bias))
    r.train()
    return r


@pytest.mark.parametrize("kind", ["qwen3", "dsv3", "glm"])
@pytest.mark.parametrize("T", [1000, 4096])
def test_fused_router_matches_tensor_operations(kind, T):
    torch.manual_seed(3)
    dev = torch.device("cuda")
    r = _router(kind, dev)
    x = torch.randn(T, 256, device=dev, dtype=torch.bfloat16)
    gw = torch.randn(T, r.top_k, device=dev)
    res = {}
    for mode in ("1", "0"):
        os.environ["PFB_FUSED_ROUTER"] = mode
        r.weight.grad = None
        r.expert_usage.zero_()
        idx, w, aux = r(x)
        loss = (w * gw).sum() + (aux if aux is not None else 0.0) * 3.0
        loss.backward()
        res[mode] = (idx, w, aux, r.weight.grad.clone(), r.expert_usage.clone(), r.last_plan)
    os.environ["PFB_FUSED_ROUTER"] = "1"
    (i1, w1, a1, g1, u1, plan), (i0, w0, a0, g0, u0, _) = res["1"], res["0"]
    assert plan is not None, "the fused path did not run"
    # the same experts per token (order inside the k may differ), the same weights per expert
    o1, o0 = i1.argsort(-1), i0.argsort(-1)
    assert torch.equal(i1.gather(1, o1), i0.gather(1, o0))
    torch.testing.assert_close(w1.gather(1, o1), w0.gather(1, o0), rtol=1e-4, atol=1e-6)
    assert torch.equal(u1, u0)
    if a0 is not None:
        torch.testing.assert_close(a1, a0, rtol=1e-4, atol=1e-7)
    rel = ((g1 - g0).norm() / (g0.norm() + 1e-12)).item()
    assert rel < 2e-3, rel
    # counts and stable ranks against a stable sort of the kernel's own pairs
    flat = i1.reshape(-1)
    counts = torch.bincount(flat, minlength=r.num_experts)
    assert torch.equal(plan["counts"].long(), counts)
    order = torch.argsort(flat, stable=True)
    first = torch.cumsum(counts, 0) - counts
    rank_sorted = torch.arange(flat.numel(), device=dev) - first[flat[order]]
    rank = torch.empty_like(rank_sorted)
    rank[order] = rank_sorted
    assert torch.equal(plan["rank_in_expert"].long(), rank)
