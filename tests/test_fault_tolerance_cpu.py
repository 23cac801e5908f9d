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


def test_checkpoint_mirror_verifies_copies_and_restores_the_newest_good_one(tmp_path):
    import json
    import os

    import torch

    from paddleformers_b200.utils import ckpt_mirror as cm

    def make(root, step, payload):
        d = root / f"checkpoint-{step}"
        (d / "optimizer").mkdir(parents=True)
        torch.save({"x": torch.full((64,), payload)}, d / "optimizer" / "shard.pt")
        (d / "trainer_state.json").write_text(json.dumps({"global_step": step}))
        return d

    store, fast, local = tmp_path / "store", tmp_path / "fast", tmp_path / "local"
    c2, c4 = make(store, 2, 2.0), make(store, 4, 4.0)
    assert cm.verify(str(c2))[0] is cm.MirrorStatus.CHECKSUM_MISSING
    cm.write_manifest(str(c2)); cm.write_manifest(str(c4))
    assert cm.verify(str(c4)) == (cm.MirrorStatus.SUCCESS, [])
    # the fast device keeps the newest verified copy only
    assert cm.backup_to_fast_device(str(c2), str(fast)) is cm.MirrorStatus.SUCCESS
    assert cm.backup_to_fast_device(str(c4), str(fast)) is cm.MirrorStatus.SUCCESS
    assert [s for s, _ in cm.list_checkpoints(str(fast))] == [4] and not os.path.exists(str(fast / "checkpoint-4.incoming"))
    # a corrupted source is refused and leaves no checkpoint behind (the copy is set aside)
    with open(c2 / "optimizer" / "shard.pt", "r+b") as f:
        f.seek(200); f.write(b"\\x00\\x01\\x02\\x03")
    st, problems = cm.verify(str(c2))
    assert st is cm.MirrorStatus.CHECKSUM_MISMATCH and "digest differs" in problems[0]
    assert cm.mirror(str(c2), str(tmp_path / "bad" / "checkpoint-2")) is cm.MirrorStatus.CHECKSUM_MISMATCH
    assert not os.path.exists(tmp_path / "bad" / "checkpoint-2") and os.path.exists(tmp_path / "bad" / "checkpoint-2.failed")
    # restore: the fast device's copy of step 4 wins; if it is damaged the persistent copy is taken; step 2 is never chosen
    st, path = cm.restore_latest([str(fast), str(store)], str(local))
    assert st is cm.MirrorStatus.SUCCESS and path == str(local / "checkpoint-4")
    assert torch.load(local / "checkpoint-4" / "optimizer" / "shard.pt")["x"][0] == 4.0
    os.remove(fast / "checkpoint-4" / "trainer_state.json")
    import shutil
    shutil.rmtree(local)
    st, path = cm.restore_latest([str(fast), str(store)], str(local))
    assert st is cm.MirrorStatus.SUCCESS and cm.verify(path)[0] is cm.MirrorStatus.SUCCESS
    shutil.rmtree(store / "checkpoint-4"); shutil.rmtree(fast)
    assert cm.restore_latest([str(fast), str(store)], str(tmp_path / "none")) == (cm.MirrorStatus.NOTHING_TO_RESTORE, None)


def test_trainer_mirrors_checkpoints_to_the_fast_device_and_resumes_from_it(tmp_path):
    import shutil

    import torch

    from paddleformers_b200 import AutoModelForCausalLM, Trainer, TrainingArguments
    from paddleformers_b200.data.synthetic import SyntheticCausalLMDataset
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.utils import ckpt_mirror as cm

    def run(steps):
        torch.manual_seed(0)
        model = AutoModelForCausalLM.from_config(named_config("tiny-llama", vocab_size=128, hidden_size=32, intermediate_size=48,
                                                              num_attention_heads=2, num_key_value_heads=1, head_dim=16))
        args = TrainingArguments(output_dir=str(tmp_path / "out"), per_device_train_batch_size=2, max_steps=steps, learning_rate=1e-3,
                                 save_steps=2, max_seq_len=32, lr_scheduler_type="constant", flash_device_path=str(tmp_path / "flash"))
        tr = Trainer(model=model, args=args, train_dataset=SyntheticCausalLMDataset(128, 32, 64, seed=0))
        tr.train(resume_from_checkpoint="auto")
        return tr

    run(4)
    assert [s for s, _ in cm.list_checkpoints(str(tmp_path / "flash"))] == [4]
    assert cm.verify(str(tmp_path / "flash" / "checkpoint-4"))[0] is cm.MirrorStatus.SUCCESS
    shutil.rmtree(tmp_path / "out")                       # the shared store is gone: the fast device still has step 4
    tr = run(6)
    assert tr.state.global_step == 6 and [h["global_step"] for h in tr.state.log_history if "loss" in h][-2:] == [5, 6]
