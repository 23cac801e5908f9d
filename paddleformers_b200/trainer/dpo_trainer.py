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


def _response_logps(logits: torch.Tensor, labels: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor, average: bool):
    lp = torch.log_softmax(logits.float(), dim=-1)
    tok = lp.gather(-1, labels.clamp(min=0).unsqueeze(-1)).squeeze(-1)
    S = labels.shape[1]
    pos = torch.arange(S, device=labels.device)[None]
    mask = (pos >= lo[:, None]) & (pos < hi[:, None]) & (labels != -100)
    s = (tok * mask).sum(-1)
    return s / mask.sum(-1).clamp(min=1) if average else s


class DPOTrainer(Trainer):
    def __init__(self, *args, ref_model: Optional[torch.nn.Module] = None, dpo_beta: float = 0.1, dpo_loss_type: str = "sigmoid",
                 dpo_label_smoothing: float = 0.0, sft_loss_ratio: float = 0.0, simpo_gamma: float = 0.5, **kw):
        super().__init__(*args, **kw)
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
            # multimodal pairs: rows 2b / 2b + 1 are example b's chosen / rejected sequence, targets on the response only
            extra = {k: inputs[k] for k in ("pixel_values", "image_grid_thw", "pixel_values_videos", "video_grid_thw", "token_type_ids")
                     if inputs.get(k) is not None}
            out = model(input_ids=inputs["input_ids"], return_logits=True, **extra)
            labels = inputs["labels"]
            S = labels.shape[1]
            lo, hi = torch.zeros(labels.shape[0], dtype=torch.long, device=labels.device), torch.full_like(labels[:, 0], S)
            lp = _response_logps(out.logits, labels, lo, hi, self.dpo["loss_type"] in ("simpo", "ipo", "or"))
            return lp[0::2], lp[1::2], out
        out = model(input_ids=inputs["input_ids"], position_ids=inputs.get("position_ids"),
                    attn_mask_startend_row_indices=inputs.get("attn_mask_startend_row_indices"), return_logits=True)
        idx = inputs["response_indexs"]
        avg = self.dpo["loss_type"] in ("simpo", "ipo", "or")
        chosen = _response_logps(out.logits, inputs["chosen_labels"], idx[:, 1], idx[:, 2], avg)
        rejected = _response_logps(out.logits, inputs["rejected_labels"], idx[:, 3], idx[:, 4], avg)
        return chosen, rejected, out

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
            nll = -_response_logps(out.logits, inputs["chosen_labels"], idx[:, 1], idx[:, 2], True).mean()
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
