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
