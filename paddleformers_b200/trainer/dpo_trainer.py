"""Direct preference optimisation trainer.

Follows paddleformers/cli/train/dpo/dpo_trainer.py:53 (``DPOTrainer``, ``get_batch_metrics`` :126): one forward of the
policy over rows that hold ``prompt+chosen`` and ``prompt+rejected`` as two packed documents, per-sequence
log-probabilities from ``response_indexs``, a frozen reference model (or, with LoRA, the same network with adapters
disabled) for the reference log-probabilities, and any of the nine preference losses.
"""
from __future__ import annotations

import contextlib
from typing import Any, Dict, Optional

import torch

from ..nn.criterion import dpo_loss
from .trainer import Trainer


class _SumOverSlices(torch.autograd.Function):
    """Sum over the ranks that hold slices of one sequence. Every rank goes on to compute the same loss from the sum and the
    ranks' parameter gradients are averaged afterwards (they count as data ranks), so the backward pass sums as well."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.clone()
        torch.distributed.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        torch.distributed.all_reduce(g, group=ctx.group)
        return g, None


def _response_logps(logits: torch.Tensor, labels: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor, average: bool,
                    positions: Optional[torch.Tensor] = None, groups=()):
    """Sum (or mean) of the label log-probabilities over positions [lo, hi) of every row. ``positions``: under context /
    segment parallelism the global position of every local token (``labels`` is then the whole row and ``logits`` this rank's
    slice); the partial sums are added up over ``groups``."""
    if positions is not None:
        labels = labels.index_select(1, positions)
    lp = torch.log_softmax(logits.float(), dim=-1)
    tok = lp.gather(-1, labels.clamp(min=0).unsqueeze(-1)).squeeze(-1)
    pos = torch.arange(labels.shape[1], device=labels.device) if positions is None else positions
    mask = (pos[None] >= lo[:, None]) & (pos[None] < hi[:, None]) & (labels != -100)
    s, n = (tok * mask).sum(-1), mask.sum(-1).to(torch.float32)
    for g in groups:
        s, n = _SumOverSlices.apply(s, g), _SumOverSlices.apply(n, g)
    return s / n.clamp(min=1) if average else s


class DPOTrainer(Trainer):
    def __init__(self, *args, ref_model: Optional[torch.nn.Module] = None, dpo_beta: float = 0.1, dpo_loss_type: str = "sigmoid",
                 dpo_label_smoothing: float = 0.0, sft_loss_ratio: float = 0.0, simpo_gamma: float = 0.5, **kw):
        super().__init__(*args, **kw)
        if self.ps.degrees.pp > 1:
            raise NotImplementedError("preference training is implemented without pipeline stages: the loss needs the log-"
                                      "probabilities of both responses of a pair at once")
        self.ref_model = ref_model
        if self.ref_model is not None:
            self.ref_model.to(self.device).eval()
            for p in self.ref_model.parameters():
                p.requires_grad_(False)
        self.dpo = dict(beta=dpo_beta, loss_type=dpo_loss_type, label_smoothing=dpo_label_smoothing,
                        sft_loss_ratio=sft_loss_ratio, simpo_gamma=simpo_gamma)
        self.last_metrics: Dict[str, float] = {}

    def _logps(self, model, inputs):
        if "preference_pairs" in inputs:
            if self.ps.degrees.cp > 1 or self.ps.degrees.sep > 1:
                raise NotImplementedError("multimodal preference pairs are implemented without context / segment parallelism")
            # multimodal pairs: rows 2b / 2b + 1 are example b's chosen / rejected sequence, targets on the response only
            extra = {k: inputs[k] for k in ("pixel_values", "image_grid_thw", "pixel_values_videos", "video_grid_thw", "token_type_ids")
                     if inputs.get(k) is not None}
            out = model(input_ids=inputs["input_ids"], return_logits=True, **extra)
            labels = inputs["labels"]
            S = labels.shape[1]
            lo, hi = torch.zeros(labels.shape[0], dtype=torch.long, device=labels.device), torch.full_like(labels[:, 0], S)
            lp = _response_logps(out.logits, labels, lo, hi, self.dpo["loss_type"] in ("simpo", "ipo", "or"))
            return lp[0::2], lp[1::2], out
        sliced = {k: inputs[k] for k in ("cp_global_positions", "cp_full_seq_len", "full_attn_mask_startend_row_indices")
                  if inputs.get(k) is not None}
        out = model(input_ids=inputs["input_ids"], position_ids=inputs.get("position_ids"),
                    attn_mask_startend_row_indices=inputs.get("attn_mask_startend_row_indices"), return_logits=True, **sliced)
        idx = inputs["response_indexs"]
        avg = self.dpo["loss_type"] in ("simpo", "ipo", "or")
        where = self._slice_positions(inputs)
        chosen = _response_logps(out.logits, inputs["chosen_labels"], idx[:, 1], idx[:, 2], avg, *where)
        rejected = _response_logps(out.logits, inputs["rejected_labels"], idx[:, 3], idx[:, 4], avg, *where)
        return chosen, rejected, out

    def _slice_positions(self, inputs):
        """(global positions of this rank's tokens, groups to sum over) under context / segment parallelism, else (None, ())."""
        ps = self.ps
        if ps.degrees.cp > 1 and ps.degrees.sep > 1:
            raise NotImplementedError("preference training combines with context OR segment parallelism, not both")
        if ps.degrees.cp > 1:
            return inputs["cp_global_positions"], (ps.group("cp"),)
        if ps.degrees.sep > 1:
            per = inputs["input_ids"].shape[1]
            r = ps.coord["sep"]
            return torch.arange(r * per, (r + 1) * per, device=inputs["input_ids"].device), (ps.group("sep"),)
        return None, ()

    def compute_loss(self, model, inputs: Dict[str, Any]):
        pc, pr, out = self._logps(model, inputs)
        rc = rr = None
        if self.dpo["loss_type"] not in ("or", "simpo"):
            with torch.no_grad():
                if self.ref_model is not None:
                    rc, rr, _ = self._logps(self.ref_model, inputs)
                else:
                    disable = getattr(model, "disable_adapters", None)
                    ctx = disable() if disable is not None else contextlib.nullcontext()
                    with ctx:
                        rc, rr, _ = self._logps(model, inputs)
        nll = None
        if self.dpo["sft_loss_ratio"] > 0 and "preference_pairs" in inputs:
            lab = inputs["labels"][0::2]
            nll = -_response_logps(out.logits[0::2], lab, torch.zeros_like(lab[:, 0]), torch.full_like(lab[:, 0], lab.shape[1]), True).mean()
        elif self.dpo["sft_loss_ratio"] > 0:
            idx = inputs["response_indexs"]
            nll = -_response_logps(out.logits, inputs["chosen_labels"], idx[:, 1], idx[:, 2], True, *self._slice_positions(inputs)).mean()
        loss, metrics = dpo_loss(pc, pr, rc, rr, chosen_nll=nll, **self.dpo)
        self.last_metrics = {k: float(v) for k, v in metrics.items()}
        accum = self.args.gradient_accumulation_steps
        out.loss = loss / accum
        out.num_tokens = None
        return out.loss, out

    def log(self, logs):
        if "loss" in logs and self.last_metrics:
            logs = dict(logs, **self.last_metrics)
        super().log(logs)
