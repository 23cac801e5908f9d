"""Tiny Llama-style decoder SFT step on CPU, single process, fp32: 10 AdamW steps, the loss decreases and the
checkpoint round-trips through safetensors (also resumable)."""
import os

import torch

from paddleformers_b200 import AutoModelForCausalLM, Trainer, TrainingArguments
from paddleformers_b200.data.synthetic import SyntheticCausalLMDataset
from paddleformers_b200.models.configuration import named_config
from paddleformers_b200.trainer.trainer_utils import get_last_checkpoint


class _Fixed(torch.utils.data.Dataset):
    def __init__(self, ds, n):
        self.ds, self.n = ds, n

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        return self.ds[i % 2]


def _make(tmp, steps, **kw):
    torch.manual_seed(0)
    cfg = named_config("tiny-llama")
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
            cfg.intermediate_size, cfg.vocab_size) == (2, 256, 4, 2, 64, 688, 32000)
    model = AutoModelForCausalLM.from_config(cfg)
    ds = _Fixed(SyntheticCausalLMDataset(32000, 128, 8, seed=0), 64)
    base = dict(output_dir=str(tmp), per_device_train_batch_size=2, max_steps=steps, learning_rate=1e-4, logging_steps=1,
                save_steps=5, max_seq_len=128, lr_scheduler_type="constant")
    base.update(kw)
    args = TrainingArguments(**base)
    return model, Trainer(model=model, args=args, train_dataset=ds)


def test_loss_decreases_and_checkpoint_roundtrip(tmp_path):
    model, tr = _make(tmp_path, 10)
    tr.train()
    losses = [h["loss"] for h in tr.state.log_history if "loss" in h]
    assert len(losses) == 10 and losses[-1] < losses[0] - 0.05
    ck = get_last_checkpoint(str(tmp_path))
    assert ck.endswith("checkpoint-10") and os.path.exists(os.path.join(ck, "model.safetensors"))
    m2 = AutoModelForCausalLM.from_pretrained(ck)
    for (n1, p1), (n2, p2) in zip(model.state_dict().items(), m2.state_dict().items()):
        assert n1 == n2 and torch.equal(p1, p2), n1
    # HF tensor names on disk (unfused q/k/v and gate/up)
    from safetensors import safe_open

    with safe_open(os.path.join(ck, "model.safetensors"), framework="pt") as f:
        keys = set(f.keys())
    assert "model.layers.0.self_attn.q_proj.weight" in keys and "model.layers.1.mlp.up_proj.weight" in keys
    assert "lm_head.weight" in keys and not any("qkv_proj" in k for k in keys)


def test_resume_reproduces_uninterrupted_run(tmp_path):
    _, full = _make(tmp_path / "a", 10)
    full.train()
    ref = [h["loss"] for h in full.state.log_history if "loss" in h]
    _, first = _make(tmp_path / "b", 5)
    first.train()
    _, second = _make(tmp_path / "b", 10)
    second.train(resume_from_checkpoint="auto")
    got = [h["loss"] for h in second.state.log_history if "loss" in h]
    assert second.state.global_step == 10
    assert all(abs(a - b) < 1e-5 for a, b in zip(ref[5:], got[-5:])), (ref[5:], got[-5:])


def test_timers_and_scalar_reports(tmp_path):
    """report_to=jsonl writes scalars; enable_timer adds per-step timer fields to the log records."""
    import json

    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.data.synthetic import SyntheticCausalLMDataset
    from paddleformers_b200.models.configuration import named_config
    from paddleformers_b200.transformers.auto import AutoModelForCausalLM

    cfg = named_config("tiny-llama", vocab_size=128, hidden_size=32, intermediate_size=64, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=16)
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float32)
    args = TrainingArguments(output_dir=str(tmp_path), per_device_train_batch_size=1, gradient_accumulation_steps=2, max_steps=3,
                             learning_rate=1e-3, logging_steps=1, save_strategy="no", max_seq_len=16, device="cpu",
                             report_to="jsonl", enable_timer=True)
    ds = SyntheticCausalLMDataset(128, 16, num_samples=16, seed=0)
    tr = Trainer(model=model, args=args, train_dataset=ds)
    tr.train()
    recs = [h for h in tr.state.log_history if "loss" in h]
    assert len(recs) == 3 and all(r["timer_forward_backward_ms"] > 0 and r["timer_optimizer_step_ms"] > 0 for r in recs)
    lines = [json.loads(l) for l in open(tmp_path / "runs" / "scalars.jsonl")]
    tags = {l["tag"] for l in lines}
    assert {"train/loss", "train/learning_rate", "train/timer_forward_backward_ms"} <= tags


def test_timers_accumulate_intervals():
    from paddleformers_b200.utils.timer import Timers

    t = Timers(use_cuda=False)
    for _ in range(3):
        with t("a"):
            pass
    info = t.info(normalizer=3)
    assert set(info) == {"a"} and info["a"] >= 0 and t.info() == {}


def test_zero_cost_checkpoint_resume_matches_uninterrupted_run(tmp_path):
    """Optimizer-shard snapshots persisted in the background, no weight export: the resumed run rebuilds the working
    weights from the fp32 master shards and continues exactly like the uninterrupted one."""
    _, full = _make(tmp_path / "a", 10)
    full.train()
    ref = [h["loss"] for h in full.state.log_history if "loss" in h]
    _, first = _make(tmp_path / "b", 5, enable_zero_cost_checkpoint=True)
    first.train()
    from paddleformers_b200.trainer.checkpoint import wait_for_pending_saves

    wait_for_pending_saves()
    ck = get_last_checkpoint(str(tmp_path / "b"))
    assert ck.endswith("checkpoint-5") and not any(f.endswith(".safetensors") for f in os.listdir(ck))
    assert os.path.exists(os.path.join(ck, "extra_state_0.pt")) and first.zcc.snapshots == 1
    _, second = _make(tmp_path / "b", 10, enable_zero_cost_checkpoint=True)
    second.train(resume_from_checkpoint="auto")
    got = [h["loss"] for h in second.state.log_history if "loss" in h]
    assert second.state.global_step == 10
    assert all(abs(a - b) < 1e-5 for a, b in zip(ref[5:], got[-5:])), (ref[5:], got[-5:])


def test_ema_tracks_master_weights_and_exports(tmp_path):
    from paddleformers_b200.trainer.ema import EMACallback, export_ema_weights

    model, tr = _make(tmp_path, 6, ema_decay=0.5, save_strategy="no")
    ema = next(cb for cb in tr.callback_handler.callbacks if isinstance(cb, EMACallback))
    tr.train()
    assert ema.num_updates == 6
    dom = tr.optimizer.domains[0]
    shadow = ema.shadow[dom.name]
    # the average lags the live weights but stays between them and the initial weights
    assert not torch.equal(shadow, dom.master) and (shadow - dom.master).abs().max() < 1e-2
    live = {k: v.clone() for k, v in model.state_dict().items()}
    out = export_ema_weights(tr, ema, str(tmp_path / "ema"))
    for k, v in model.state_dict().items():          # the live weights are restored after the export
        assert torch.equal(v, live[k]), k
    m2 = AutoModelForCausalLM.from_pretrained(out)
    diffs = [(m2.state_dict()[k].float() - live[k].float()).abs().max().item() for k in live]
    assert max(diffs) > 0 and max(diffs) < 1e-2


def test_zero_cost_checkpoint_ema_flags_average_on_an_interval_and_below_a_loss_threshold(tmp_path):
    from paddleformers_b200.trainer.ema import EMACallback

    _, tr = _make(tmp_path, 6, enable_zero_cost_checkpoint=True, zcc_save_ema_coef=0.5, zcc_ema_interval=2, save_strategy="no")
    ema = next(cb for cb in tr.callback_handler.callbacks if isinstance(cb, EMACallback))
    tr.train()
    assert ema.decay == 0.5 and ema.num_updates == 3              # steps 2, 4, 6
    _, tr = _make(tmp_path, 4, enable_zero_cost_checkpoint=True, zcc_save_ema_coef=0.5, zcc_ema_loss_threshold=1e-3,
                  save_strategy="no")
    ema = next(cb for cb in tr.callback_handler.callbacks if isinstance(cb, EMACallback))
    tr.train()
    assert ema.num_updates <= 1                                   # the loss never gets below the threshold once it is known


def test_muon_orthogonalises_matrix_updates_and_trains(tmp_path):
    from paddleformers_b200.parallel.sharding import ShardedMuon, newton_schulz_orthogonalize

    torch.manual_seed(0)
    G = torch.randn(48, 80)
    sv = torch.linalg.svdvals(newton_schulz_orthogonalize(G))
    assert sv.min() > 0.5 and sv.max() < 1.3                       # all singular values pushed towards one
    _, tr = _make(tmp_path, 8, optim="muon", save_strategy="no", learning_rate=2e-3)
    tr.train()
    assert isinstance(tr.optimizer, ShardedMuon)
    names = {d.name: [n for n, _ in d.params] for d in tr.optimizer.domains}
    muon = [n for k, v in names.items() if k.endswith("_muon") for n in v]
    adam = [n for k, v in names.items() if not k.endswith("_muon") for n in v]
    assert any("qkv_proj" in n for n in muon) and any("down_proj" in n for n in muon)
    assert any("embed_tokens" in n for n in adam) and any("norm" in n for n in adam) and not any("embed" in n for n in muon)
    losses = [h["loss"] for h in tr.state.log_history if "loss" in h]
    assert losses[-1] < losses[0] - 0.05


def test_torch_profiler_window_writes_trace(tmp_path):
    from paddleformers_b200.utils.profiler import StartupTimer

    _, tr = _make(tmp_path, 4, save_strategy="no", profile=True, profile_backend="torch", profile_step_start=1, profile_step_end=3)
    tr.train()
    prof_dir = tmp_path / "profile"
    assert (prof_dir / "trace_rank0.json").stat().st_size > 1000 and "Name" in (prof_dir / "top_ops_rank0.txt").read_text()
    st = StartupTimer()
    st.mark("imports"); st.mark("model")
    assert "imports" in st.report()


def test_two_runs_with_one_seed_agree_bit_for_bit(tmp_path, monkeypatch):
    """Run-to-run determinism, checked through the loss digests of the log records; a different seed changes them."""
    from paddleformers_b200.trainer.trainer_utils import state_digest, tensor_md5

    def run(sub, seed):
        m, tr = _make(tmp_path / sub, 4, save_strategy="no", log_loss_md5=True, seed=seed)
        tr.train()
        return [h["loss_md5"] for h in tr.state.log_history if "loss_md5" in h], state_digest(dict(m.state_dict()))

    a, da = run("a", 1)
    b, db = run("b", 1)
    assert len(a) == 4 and all(len(x) == 32 for x in a)
    assert a == b and da == db
    # the digest is of the fp32 bit pattern, so the smallest change shows
    x = torch.tensor([1.0])
    assert tensor_md5(x) != tensor_md5(torch.nextafter(x, torch.tensor([2.0])))
    assert tensor_md5(x.bfloat16()) == tensor_md5(x)
    # the environment switch does the same as the argument
    monkeypatch.setenv("LOG_LOSS_MD5", "1")
    _, tr = _make(tmp_path / "c", 1, save_strategy="no")
    tr.train()
    assert "loss_md5" in tr.state.log_history[0]


def test_module_ranges_nest_and_balance_in_forward_and_backward():
    from paddleformers_b200.utils.profiler import NvtxModuleRanges

    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(named_config("tiny-llama"))
    events, stack = [], []

    def push(label):
        stack.append(label)
        events.append(("push", label, len(stack)))

    def pop():
        events.append(("pop", stack.pop(), len(stack)))

    ids = torch.randint(0, 32000, (1, 16))
    with NvtxModuleRanges(model, depth=3, push=push, pop=pop) as ranges:
        assert ranges.handles
        out = model(input_ids=ids, labels=ids)
        loss = out[0] if isinstance(out, tuple) else out.loss
        assert not stack                     # every forward range closed
        loss.backward()
        assert not stack                     # every backward range closed
    pushed = [e[1] for e in events if e[0] == "push"]
    assert any(l.startswith("model.layers.0:") for l in pushed) and any(l.startswith("model.layers.1:") for l in pushed)
    assert any(l.startswith("bwd:model.layers.0:") for l in pushed)
    assert max(e[2] for e in events) >= 2     # children open inside their parent's range
    assert not any(l.count(".") >= 3 for l in (x.split(":")[-2] if x.startswith("bwd:") else x.split(":")[0] for x in pushed))
    n = len(events)
    model(input_ids=ids)                      # hooks removed on exit
    assert len(events) == n


def test_best_checkpoint_is_tracked_and_reloaded_at_the_end(tmp_path):
    """load_best_model_at_end: the checkpoint of the step with the lowest evaluation loss is remembered and its weights are
    back in the model when train() returns; max_evaluate_steps bounds the evaluation; the scheduler takes power / lr_end."""
    torch.manual_seed(0)
    cfg = named_config("tiny-llama")
    model = AutoModelForCausalLM.from_config(cfg)
    train = _Fixed(SyntheticCausalLMDataset(32000, 128, 8, seed=0), 64)
    evals = _Fixed(SyntheticCausalLMDataset(32000, 128, 8, seed=0), 8)
    args = TrainingArguments(output_dir=str(tmp_path), per_device_train_batch_size=2, max_steps=6, learning_rate=3e-4, logging_steps=1,
                             save_steps=2, eval_strategy="steps", eval_steps=2, max_evaluate_steps=2, max_seq_len=128,
                             lr_scheduler_type="polynomial", power=2.0, lr_end=1e-5, load_best_model_at_end=True)
    assert args.min_lr == 1e-5
    tr = Trainer(model=model, args=args, train_dataset=train, eval_dataset=evals)
    tr.train()
    evs = [h for h in tr.state.log_history if "eval_loss" in h]
    assert len(evs) == 3 and all(h["eval_steps_per_second"] > 0 for h in evs)
    best = min(range(3), key=lambda i: evs[i]["eval_loss"])
    assert tr.state.best_metric == evs[best]["eval_loss"]
    assert tr.state.best_model_checkpoint.endswith(f"checkpoint-{2 * (best + 1)}")
    ref = AutoModelForCausalLM.from_pretrained(tr.state.best_model_checkpoint)
    for (n1, p1), (n2, p2) in zip(model.state_dict().items(), ref.state_dict().items()):
        assert torch.equal(p1, p2), n1
