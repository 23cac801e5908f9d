"""Command line: argument parsing, unknown-key errors, a full PT run from a YAML config, launch command."""
import json
import os

import numpy as np
import pytest
import torch


def test_parse_overrides_and_unknown_keys(tmp_path):
    from paddleformers_b200.cli.hparams import get_train_args

    cfg = tmp_path / "c.yaml"
    cfg.write_text("stage: SFT\nmodel_type: tiny-llama\nlearning_rate: 1.0e-3\nlora: true\ncompute_type: float32\n"
                   "tensor_model_parallel_size: 1\noutput_dir: %s\n" % tmp_path)
    m, d, g, e, t = get_train_args([str(cfg), "lora_rank=4", "max_steps=3", "packing=false"])
    assert m.lora and m.lora_rank == 4 and t.max_steps == 3 and t.learning_rate == 1e-3 and d.packing is False
    assert t.bf16 is False and t.data_parallel_size == 1
    with pytest.raises(ValueError, match="unknown configuration keys"):
        get_train_args([str(cfg), "not_a_flag=1"])


@pytest.mark.parametrize("stage", ["PT", "auto-parallel"])
def test_pretrain_stage_end_to_end_from_yaml(tmp_path, stage):
    from paddleformers_b200.cli.cli import main
    from paddleformers_b200.data.indexed_dataset import MMapIndexedDatasetBuilder

    prefix = str(tmp_path / "corpus")
    b = MMapIndexedDatasetBuilder(prefix, dtype=np.uint16)
    rng = np.random.RandomState(0)
    for _ in range(64):
        b.add_document(rng.randint(2, 120, size=rng.randint(20, 60)))
    b.finalize()
    out = tmp_path / "out"
    cfg = tmp_path / "pt.json"
    cfg.write_text(json.dumps({
        "stage": stage, "model_type": "tiny-llama", "from_scratch": True, "compute_type": "float32", "device": "cpu",
        "config_overrides": {"vocab_size": 128, "hidden_size": 32, "intermediate_size": 48, "num_attention_heads": 2,
                             "num_key_value_heads": 1, "head_dim": 16},
        "input_dir": prefix, "split": "9,1,0", "max_seq_len": 32, "max_steps": 4, "per_device_train_batch_size": 2,
        "learning_rate": 1e-3, "logging_steps": 1, "save_strategy": "no", "output_dir": str(out)}))
    env = os.environ.pop("CUDA_VISIBLE_DEVICES", None)
    os.environ["CUDA_VISIBLE_DEVICES"] = ""
    try:
        assert main(["train", str(cfg)]) == 0
    finally:
        if env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = env
    assert os.path.exists(out / "model.safetensors") and os.path.exists(out / "config.json")


def test_launch_command_uses_loopback_rendezvous(monkeypatch):
    from paddleformers_b200.cli.cli import build_launch_command

    monkeypatch.delenv("MASTER_ADDR", raising=False)
    cmd = build_launch_command(["cfg.yaml", "a=1"], 8)
    assert "--nproc-per-node=8" in cmd and "--master-addr=127.0.0.1" in cmd and cmd[-2:] == ["cfg.yaml", "a=1"]
