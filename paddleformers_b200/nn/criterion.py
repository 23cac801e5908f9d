"""Loss functions: SFT cross entropy, multi-token-prediction weighting, DPO family, KTO.

Counterparts: paddleformers/nn/criterion/interface.py:40-91 (``CriterionLayer``), sft_loss.py:44-57 (masked mean in
fp32 returning (loss, loss_sum)), dpo_loss.py:248-333 (nine preference losses), kto_loss.py.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as TF

IGNORE_INDEX = -100


def sft_loss(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = IGNORE_INDEX) -> Tuple[torch.Tensor, torch.Tensor]:
    """(mean over non-ignored tokens, sum) of the token cross entropy, computed in fp32."""
    tok = TF.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), labels.reshape(-1), ignore_index=ignore_index, reduction="none")
    mask = (labels.reshape(-1) != ignore_index).float()
    s = (tok * mask).sum()
    return s / mask.sum().clamp(min=1.0), s


def sequence_logps(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = IGNORE_INDEX, average: bool = False):
    """Sum (or mean) of the log-probabilities of the labelled tokens per row."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    mask = labels != ignore_index
    tok = lp.gather(-1, labels.clamp(min=0).unsqueeze(-1)).squeeze(-1) * mask
    s = tok.sum(-1)
    return s / mask.sum(-1).clamp(min=1) if average else s


DPO_LOSS_TYPES = ("sigmoid", "hinge", "ipo", "kto_pair", "sppo_hard", "nca_pair", "dpop", "or", "simpo")


def dpo_loss(policy_chosen: torch.Tensor, policy_rejected: torch.Tensor, ref_chosen: Optional[torch.Tensor],
             ref_rejected: Optional[torch.Tensor], loss_type: str = "sigmoid", beta: float = 0.1, label_smoothing: float = 0.0,
             simpo_gamma: float = 0.5, dpop_lambda: float = 50.0, sft_loss_ratio: float = 0.0,
             chosen_nll: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """Preference losses on per-sequence log-probabilities. ``or`` (ORPO) and ``simpo`` are reference-free."""
    if loss_type not in DPO_LOSS_TYPES:
        raise ValueError(f"unknown dpo loss {loss_type!r}; choose from {DPO_LOSS_TYPES}")
    if loss_type in ("or", "simpo"):
        ref_chosen = torch.zeros_like(policy_chosen) if ref_chosen is None else ref_chosen
        ref_rejected = torch.zeros_like(policy_rejected) if ref_rejected is None else ref_rejected
    pi = policy_chosen - policy_rejected
    ref = ref_chosen - ref_rejected
    logits = pi - ref
    if loss_type == "sigmoid":
        loss = -TF.logsigmoid(beta * logits) * (1 - label_smoothing) - TF.logsigmoid(-beta * logits) * label_smoothing
    elif loss_type == "hinge":
        loss = torch.relu(1 - beta * logits)
    elif loss_type == "ipo":
        loss = (logits - 1 / (2 * beta)) ** 2
    elif loss_type == "kto_pair":
        ck = (policy_chosen - ref_chosen).mean().clamp(min=0)
        rk = (policy_rejected - ref_rejected).mean().clamp(min=0)
        loss = torch.cat([1 - torch.sigmoid(beta * ((policy_chosen - ref_chosen) - rk)),
                          1 - torch.sigmoid(beta * (ck - (policy_rejected - ref_rejected)))], 0)
    elif loss_type == "sppo_hard":
        a, b = policy_chosen - ref_chosen, policy_rejected - ref_rejected
        loss = (a - 0.5 / beta) ** 2 + (b + 0.5 / beta) ** 2
    elif loss_type == "nca_pair":
        cr, rr = (policy_chosen - ref_chosen) * beta, (policy_rejected - ref_rejected) * beta
        loss = -TF.logsigmoid(cr) - 0.5 * TF.logsigmoid(-cr) - 0.5 * TF.logsigmoid(-rr)
    elif loss_type == "dpop":
        penalty = torch.relu(ref_chosen - policy_chosen)
        loss = -TF.logsigmoid(beta * (logits - dpop_lambda * penalty))
    elif loss_type == "or":
        log_odds = (policy_chosen - policy_rejected) - (torch.log1p(-torch.exp(policy_chosen).clamp(max=1 - 1e-7)) -
                                                         torch.log1p(-torch.exp(policy_rejected).clamp(max=1 - 1e-7)))
        loss = -beta * TF.logsigmoid(log_odds)
    else:  # simpo (expects length-averaged log-probabilities)
        loss = -TF.logsigmoid(beta * pi - simpo_gamma)
    loss = loss.mean()
    if sft_loss_ratio > 0 and chosen_nll is not None:
        loss = loss + sft_loss_ratio * chosen_nll
    metrics = {
        "rewards/chosen": (beta * (policy_chosen - ref_chosen)).detach().mean(),
        "rewards/rejected": (beta * (policy_rejected - ref_rejected)).detach().mean(),
        "rewards/accuracies": (pi > ref).float().mean().detach(),
        "rewards/margins": (beta * logits).detach().mean(),
    }
    return loss, metrics


def kto_loss(policy_logps, ref_logps, is_desirable: torch.Tensor, kl: torch.Tensor, beta: float = 0.1,
             desirable_weight: float = 1.0, undesirable_weight: float = 1.0):
    """Kahneman-Tversky optimisation on unpaired examples; ``kl`` is the batch estimate of KL(policy || reference)."""
    r = policy_logps - ref_logps
    kl = kl.detach().clamp(min=0)
    good = 1 - torch.sigmoid(beta * (r - kl))
    bad = 1 - torch.sigmoid(beta * (kl - r))
    loss = torch.where(is_desirable.bool(), desirable_weight * good, undesirable_weight * bad)
    return loss.mean()


class CriterionLayer(torch.nn.Module):
    """Picks the loss by name, like the reference's registry ("sft" | "dpo" | "kto")."""

    def __init__(self, loss_type: str = "sft", **kw):
        super().__init__()
        self.loss_type, self.kw = loss_type, kw

    def forward(self, *args, **kwargs):
        if self.loss_type == "sft":
            return sft_loss(*args, **kwargs)
        if self.loss_type == "dpo":
            return dpo_loss(*args, **{**self.kw, **kwargs})
        if self.loss_type == "kto":
            return kto_loss(*args, **{**self.kw, **kwargs})
        raise ValueError(self.loss_type)
