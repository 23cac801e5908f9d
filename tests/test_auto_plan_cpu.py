"""Analytic parallelism planner."""
import pytest

from paddleformers_b200.models.configuration import LlamaConfig, named_config
from paddleformers_b200.parallel.auto_plan import count_parameters, estimate_memory_gb, plan_parallelism
from paddleformers_b200.parallel.topology import ParallelDegrees


def test_parameter_counts():
    n = count_parameters(named_config("llama3-8b"))
    assert abs(n["dense"] - 8.03e9) < 0.02e9 and n["expert"] == 0
    q = count_parameters(named_config("qwen3-30b-a3b"))
    assert abs(q["dense"] + q["expert"] - 30.5e9) < 0.3e9 and q["expert"] > 10 * q["dense"]


def test_plans_prefer_cheap_axes_and_fit():
    llama = named_config("llama3-8b")
    p1 = plan_parallelism(llama, 1, 4096)
    assert (p1.degrees.mp, p1.degrees.pp, p1.degrees.sharding) == (1, 1, 1) and p1.memory_gb < 162
    p8 = plan_parallelism(llama, 8, 4096)
    assert (p8.degrees.mp, p8.degrees.sharding) == (1, 8)                 # fits without model parallelism: shard the optimizer
    qwen = plan_parallelism(named_config("qwen3-30b-a3b"), 8, 4096)
    assert qwen.degrees.ep == 8 and qwen.degrees.mp == 1 and qwen.training_args()["expert_model_parallel_size"] == 8
    l70 = LlamaConfig(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                      num_attention_heads=64, num_key_value_heads=8, head_dim=128)
    p70 = plan_parallelism(l70, 16, 4096)
    assert p70.degrees.mp * p70.degrees.pp > 1 and p70.memory_gb < 162
    with pytest.raises(ValueError, match="no parallel configuration fits"):
        plan_parallelism(l70, 2, 4096)


def test_memory_estimate_scales_with_axes():
    cfg = named_config("llama3-8b")
    base = estimate_memory_gb(cfg, ParallelDegrees(), 4096)
    tp2 = estimate_memory_gb(cfg, ParallelDegrees(mp=2), 4096)
    sh2 = estimate_memory_gb(cfg, ParallelDegrees(sharding=2), 4096)
    assert tp2["weights"] == pytest.approx(base["weights"] / 2) and tp2["activations"] == pytest.approx(base["activations"] / 2)
    assert sh2["optimizer"] == pytest.approx(base["optimizer"] / 2) and sh2["weights"] == pytest.approx(base["weights"])
