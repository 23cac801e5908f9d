"""Failure detection without touching a GPU: lost ranks via heartbeats, collective timeouts on gloo ranks, interrupted
checkpoints, restart-from-last-checkpoint."""
import os
import sys
import time

import pytest
import torch

from dist_utils import run_distributed


def test_heartbeat_reports_silent_rank():
    from torch.distributed import HashStore

    from paddleformers_b200.utils.fault_tolerance import HeartbeatMonitor, RankLostError

    store = HashStore()
    a = HeartbeatMonitor(store, 0, 3, timeout_s=0.2)
    b = HeartbeatMonitor(store, 1, 3, timeout_s=0.2)
    a.beat(); b.beat()
    assert a.silent_ranks() == [2]          # rank 2 never joined
    c = HeartbeatMonitor(store, 2, 3, timeout_s=0.2)
    c.beat()
    assert a.silent_ranks() == []
    time.sleep(0.3)
    a.beat(); c.beat()                       # rank 1 stops beating
    with pytest.raises(RankLostError, match="ranks \\[1\\]"):
        a.check()


def _rank_that_leaves(rank, world):
    """Rank 1 exits between steps; rank 0 learns of it through a short process-group timeout instead of hanging."""
    import datetime

    import torch.distributed as dist

    g = dist.new_group(ranks=[0, 1], timeout=datetime.timedelta(seconds=2))
    t = torch.ones(1)
    dist.all_reduce(t, group=g)              # step 1: both alive
    if rank == 1:
        return "left"
    try:
        dist.all_reduce(t, group=g)
        return "no error"
    except Exception as e:  # noqa: BLE001
        return "detected: " + type(e).__name__


def test_lost_rank_ends_collective_with_error():
    # rank 1 returns early (its process stays in the final barrier of the harness, never joining the collective)
    from dist_utils import _free_port  # noqa: F401

    import torch.multiprocessing as mp

    res = None
    try:
        res = run_distributed(_rank_that_leaves, 2, timeout=60)
    except RuntimeError as e:
        # the surviving rank may also fail inside the harness barrier: the error must be a reported one, not a hang
        assert "failed" in str(e) or "did not exit" in str(e) or "no result" in str(e)
        return
    assert res[1] == "left" and res[0].startswith("detected")


def test_incomplete_checkpoint_is_skipped(tmp_path):
    from paddleformers_b200.trainer.trainer_utils import checkpoint_is_complete, get_last_checkpoint

    good, bad = tmp_path / "checkpoint-5", tmp_path / "checkpoint-10"
    for d in (good, bad):
        os.makedirs(d)
        (d / "model.safetensors").write_bytes(b"x")
    (good / ".checkpoint_done").write_text("1")
    (bad / "save_meta.json").write_text('{"num_writers": 2}')
    (bad / "saved_signal_0").write_text("done")     # rank 1 never finished
    assert checkpoint_is_complete(str(good)) and not checkpoint_is_complete(str(bad))
    assert get_last_checkpoint(str(tmp_path)).endswith("checkpoint-5")
    (bad / "saved_signal_1").write_text("done")
    assert get_last_checkpoint(str(tmp_path)).endswith("checkpoint-10")


def test_run_with_restarts(tmp_path):
    from paddleformers_b200.utils.fault_tolerance import run_with_restarts

    marker = tmp_path / "count"
    script = tmp_path / "job.py"
    script.write_text(
        "import os, sys\n"
        f"p = {str(marker)!r}\n"
        "n = int(open(p).read()) if os.path.exists(p) else 0\n"
        "open(p, 'w').write(str(n + 1))\n"
        "sys.exit(0 if n >= 2 else 17)\n")
    seen = []
    rc = run_with_restarts([sys.executable, str(script)], str(tmp_path), max_restarts=5, on_restart=lambda a, c: seen.append((a, c)))
    assert rc == 0 and seen == [(1, 17), (2, 17)] and marker.read_text() == "3"


def test_nonfinite_loss_raises_named_error(tmp_path):
    from paddleformers_b200 import AutoModelForCausalLM, Trainer, TrainingArguments
    from paddleformers_b200.data.synthetic import SyntheticCausalLMDataset
    from paddleformers_b200.models.configuration import named_config

    torch.manual_seed(0)
    cfg = named_config("tiny-llama", vocab_size=64, hidden_size=32, intermediate_size=48, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=16)
    model = AutoModelForCausalLM.from_config(cfg)
    with torch.no_grad():
        model.model.norm.weight.fill_(float("nan"))   # NaN injected through a tensor on the host, not a kernel trap
    tr = Trainer(model=model, args=TrainingArguments(output_dir=str(tmp_path), max_steps=2, save_strategy="no", max_seq_len=16),
                 train_dataset=SyntheticCausalLMDataset(64, 16, 8))
    with pytest.raises(FloatingPointError, match="LOSS_NAN_ERROR"):
        tr.train()
