"""Evaluation loop: whole-set coverage (also when the set does not divide into batches), token-weighted loss over data ranks,
``compute_metrics`` on gathered predictions, several evaluation sets, ``predict``."""
import math

import pytest
import torch

from dist_utils import run_distributed


def _cfg():
    from paddleformers_b200.models.configuration import named_config

    return named_config("tiny-llama", num_hidden_layers=2, hidden_size=32, intermediate_size=48, num_attention_heads=2,
                        num_key_value_heads=2, head_dim=16, vocab_size=64)


class _DS(torch.utils.data.Dataset):
    def __init__(self, n, seed=0, labels=True):
        g = torch.Generator().manual_seed(seed)
        self.rows = []
        for i in range(n):
            S = 6 + i % 5                                   # rows of different lengths: the collator pads
            ids = torch.randint(1, 64, (S + 1,), generator=g)
            row = {"input_ids": ids[:-1]}
            if labels:
                row["labels"] = ids[1:].clone()
            self.rows.append(row)

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]


def _collate(batch):
    S = max(len(b["input_ids"]) for b in batch)
    out = {"input_ids": torch.zeros(len(batch), S, dtype=torch.long)}
    if "labels" in batch[0]:
        out["labels"] = torch.full((len(batch), S), -100, dtype=torch.long)
    for i, b in enumerate(batch):
        out["input_ids"][i, :len(b["input_ids"])] = b["input_ids"]
        if "labels" in b:
            out["labels"][i, :len(b["labels"])] = b["labels"]
    return out


def _reference_loss(model, ds):
    tot, cnt = 0.0, 0
    model.eval()
    with torch.no_grad():
        for row in ds.rows:
            out = model(row["input_ids"][None], labels=row["labels"][None])
            n = int((row["labels"] != -100).sum())
            tot += out.loss.item() * n
            cnt += n
    return tot / cnt


def _worker(rank, world, state):
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.modeling import MODEL_MAPPING

    args = TrainingArguments(output_dir="/tmp/pfb_eval_unused", per_device_eval_batch_size=3, device="cpu", save_strategy="no")
    args.setup_parallel()
    cfg = _cfg()
    model = MODEL_MAPPING[cfg.model_type](cfg)
    model.load_state_dict(state)
    seen = {}

    def metrics(p):
        seen["shape"] = (p.predictions.shape, p.label_ids.shape)
        mask = p.label_ids != -100
        return {"accuracy": float(((p.predictions == p.label_ids) & mask).sum() / mask.sum()), "rows": p.predictions.shape[0]}

    tr = Trainer(model=model, args=args, data_collator=_collate, eval_dataset=_DS(10), compute_metrics=metrics)
    m = tr.evaluate()
    return m, seen["shape"]


def test_whole_set_loss_metrics_and_several_sets():
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.trainer.trainer_utils import EvalSampler

    s = EvalSampler(10, rank=1, world=2, batch=3)          # 2 global batches of 6: positions 3..5 and 9..11 -> 9, then fill-ins
    assert list(s) == [3, 4, 5, 9, 0, 1] and s.padding_rows(0) == [] and s.padding_rows(1) == [1, 2]
    torch.manual_seed(0)
    cfg = _cfg()
    model = MODEL_MAPPING[cfg.model_type](cfg)
    ds = _DS(10)
    want = _reference_loss(model, ds)
    args = TrainingArguments(output_dir="/tmp/pfb_eval_unused", per_device_eval_batch_size=4, device="cpu", save_strategy="no")

    def metrics(p):
        assert p.predictions.shape == p.label_ids.shape and p.predictions.shape in ((10, 10), (5, 10))
        return {"rows": p.predictions.shape[0]}

    tr = Trainer(model=model, args=args, data_collator=_collate, eval_dataset=ds, compute_metrics=metrics)
    m = tr.evaluate()
    assert m["eval_loss"] == pytest.approx(want, rel=1e-5) and m["eval_rows"] == 10 and m["eval_ppl"] == pytest.approx(math.exp(want), rel=1e-4)
    both = tr.evaluate({"a": ds, "b": _DS(5, seed=1)})
    assert both["eval_a_loss"] == pytest.approx(want, rel=1e-5) and "eval_b_loss" in both and both["eval_b_rows"] == 5
    # predict: with labels -> loss too; without -> predictions only; custom post-processing of the logits
    out = tr.predict(ds)
    assert out.predictions.shape == (10, 10) and out.metrics["test_loss"] == pytest.approx(want, rel=1e-5)
    tr.preprocess_logits_for_metrics = lambda logits, labels: logits.float().max(-1).values.mean(-1)      # one score per row
    scores = tr.predict(_DS(7, seed=2, labels=False))
    assert scores.predictions.shape == (7,) and scores.label_ids is None and "test_loss" not in scores.metrics
    # two data ranks see the same set: same loss, predictions back in dataset order
    state = {k: v.clone() for k, v in model.state_dict().items()}
    got = run_distributed(_worker, 2, state)
    for m2, shape in got:
        assert m2["eval_loss"] == pytest.approx(want, rel=1e-5) and m2["eval_rows"] == 10 and shape == ((10, 10), (10, 10))
    assert got[0][0]["eval_accuracy"] == got[1][0]["eval_accuracy"]


def _strategy_worker(rank, world, kind, targs, full, pipeline):
    import numpy as np

    import test_parallel_cpu as T
    from paddleformers_b200 import Trainer, TrainingArguments
    from paddleformers_b200.models.modeling import MODEL_MAPPING
    from paddleformers_b200.parallel.pipeline import build_pipeline_model
    from paddleformers_b200.transformers.configuration_utils import LlmMetaConfig
    from paddleformers_b200.transformers.model_utils import param_shard_spec

    args = TrainingArguments(output_dir="/tmp/pfb_test_unused", per_device_train_batch_size=1, per_device_eval_batch_size=1,
                             max_steps=1, logging_steps=1, save_strategy="no", max_seq_len=32, seed=3, device="cpu", **targs)
    ps = args.setup_parallel()
    cfg = T._tiny_cfg(kind, num_hidden_layers=4)
    LlmMetaConfig.set_llm_config(cfg, args)
    model = build_pipeline_model(cfg) if pipeline else MODEL_MAPPING[cfg.model_type](cfg)
    with torch.no_grad():
        for name, p in model.named_parameters():
            g = model.global_param_name(name) if pipeline else name
            p.copy_(param_shard_spec(p).shard(full[g], ps.coord["mp"], ps.degrees.mp, ps.rank_in("ep"), ps.degrees.ep))

    def metrics(p):
        pred, lab = np.asarray(p.predictions), np.asarray(p.label_ids)
        return {"hits": float(((pred == lab) & (lab != -100)).sum()), "labelled": float((lab != -100).sum()),
                "checksum": float((pred * (lab != -100)).sum())}

    data = T._DS(T._data(6))
    tr = Trainer(model=model, args=args, train_dataset=data, eval_dataset=data, compute_metrics=None if pipeline else metrics)
    return {k: round(float(v), 5) for k, v in tr.evaluate().items() if k in ("eval_loss", "eval_hits", "eval_labelled", "eval_checksum")}


@pytest.mark.parametrize("name,world,kind,targs", [
    ("tied_tp2_sp", 2, "tied", dict(tensor_model_parallel_size=2, sequence_parallel=True)),
    ("cp2", 2, False, dict(context_parallel_size=2)),
    ("sep2", 2, False, dict(sep_parallel_size=2)),
    ("pp2_interleaved", 2, False, dict(pipeline_model_parallel_size=2, virtual_pipeline_model_parallel_size=2, gradient_accumulation_steps=2)),
    ("pp2_zbv", 2, False, dict(pipeline_model_parallel_size=2, pipeline_schedule="zbv", gradient_accumulation_steps=2)),
    ("pp2_cp2", 4, False, dict(pipeline_model_parallel_size=2, context_parallel_size=2, gradient_accumulation_steps=2)),
])
def test_evaluation_under_parallel_strategies(name, world, kind, targs):
    """Loss, and where the logits exist the predictions, equal the single-process evaluation: vocabulary shards are
    concatenated, sequence slices are put back at their global positions and their losses combined, pipeline stages run a
    forward-only pass and report the loss."""
    import test_parallel_cpu as T
    from paddleformers_b200.models.modeling import MODEL_MAPPING

    torch.manual_seed(5)
    cfg = T._tiny_cfg(kind, num_hidden_layers=4)
    full = {k: v.detach().clone() for k, v in MODEL_MAPPING[cfg.model_type](cfg).named_parameters()}
    ref = run_distributed(_strategy_worker, 1, kind, {}, full, False)[0]
    got = run_distributed(_strategy_worker, world, kind, targs, full, name.startswith("pp2"))
    for r in range(world):
        for k, v in got[r].items():
            assert abs(v - ref[k]) < 1e-4 * max(1.0, abs(ref[k])), (name, r, ref, got[r])
        assert ("eval_hits" in got[r]) == (not name.startswith("pp2"))
