"""Refined recompute: named operations keep their saved tensors under per-layer recompute and are not run again."""
import pytest
import torch

from paddleformers_b200.models.configuration import named_config
from paddleformers_b200.models.modeling import MODEL_MAPPING
from paddleformers_b200.utils import refined_recompute as rr


def _model(**kw):
    torch.manual_seed(0)
    cfg = named_config("tiny-llama", num_hidden_layers=4, hidden_size=64, intermediate_size=96, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, vocab_size=128, **kw)
    return MODEL_MAPPING[cfg.model_type](cfg).train()


def _grads(model, ids, labels):
    model.zero_grad()
    out = model(ids, labels=labels)
    out.loss.backward()
    return out.loss.item(), {n: p.grad.clone() for n, p in model.named_parameters()}


def test_kept_operations_run_once_and_gradients_do_not_change():
    ids = torch.randint(0, 128, (2, 24))
    labels = torch.randint(0, 128, (2, 24))
    base = _model()
    loss0, g0 = _grads(base, ids, labels)
    full = _model(recompute_granularity="full")
    loss1, g1 = _grads(full, ids, labels)
    refined = _model(recompute_granularity="full", refined_recompute={"flash_attn": 0, "mlp_column_ln": 2, "attention_row_ln": -1})
    calls = {"attn": 0}
    from paddleformers_b200.ops import functional as F

    orig = F.flash_attention_qkvpacked

    def counting(*a, **k):
        calls["attn"] += 1
        return orig(*a, **k)

    F.flash_attention_qkvpacked = counting
    rr.STATS.update(kept=0, reused=0)
    try:
        loss2, g2 = _grads(refined, ids, labels)
    finally:
        F.flash_attention_qkvpacked = orig
    assert loss0 == pytest.approx(loss1, abs=1e-6) and loss0 == pytest.approx(loss2, abs=1e-6)
    for n in g0:
        assert torch.allclose(g0[n], g1[n], atol=1e-6) and torch.allclose(g0[n], g2[n], atol=1e-6), n
    # attention kept in all 4 layers (4 calls instead of 8); the gate / up projection kept in the first 2 layers
    assert calls["attn"] == 4
    assert rr.STATS["kept"] == 4 + 2 and rr.STATS["reused"] == 4 + 2


def test_layer_selection_rule():
    spec = {"flash_attn": 0, "mlp_row_ln": 3, "attention_column_ln": -1}
    assert rr.kept_ops_of_layer(spec, 0, 8) == {"flash_attn", "mlp_row_ln"}
    assert rr.kept_ops_of_layer(spec, 4, 8) == {"flash_attn", "mlp_row_ln"}
    assert rr.kept_ops_of_layer(spec, 5, 8) == {"flash_attn"}                   # the last 3 layers recompute the down projection
    # a pipeline stage that holds layers 4..7 of 8 keeps it in its first ceil(4 * 5 / 8) = 3 layers
    assert [("mlp_row_ln" in rr.kept_ops_of_layer(spec, i, 8, [4, 5, 6, 7])) for i in (4, 5, 6, 7)] == [True, True, True, False]
    with pytest.raises(ValueError, match="unknown operation"):
        rr.kept_ops_of_layer({"softmax": 1}, 0, 8)


def test_outside_a_frame_and_without_gradients_keep_is_a_plain_call():
    x = torch.randn(3, 4, requires_grad=True)
    assert torch.equal(rr.keep("flash_attn", torch.relu, x), torch.relu(x))
    m = _model(recompute_granularity="full", refined_recompute={"flash_attn": 0}).eval()
    with torch.no_grad():
        m(torch.randint(0, 128, (1, 8)))
    assert getattr(rr._local, "frame", None) is None


def test_flag_reaches_the_model_through_the_training_arguments(tmp_path):
    from paddleformers_b200 import TrainingArguments
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig

    args = TrainingArguments(output_dir=str(tmp_path), device="cpu", recompute_granularity="full", refined_recompute={"flash_attn": 0})
    cfg = named_config("tiny-llama", num_hidden_layers=2)
    LlmMetaConfig.set_llm_config(cfg, args)
    assert cfg.refined_recompute == {"flash_attn": 0} and cfg.recompute_granularity == "full"
