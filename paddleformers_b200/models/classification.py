"""Classification heads on the unified decoder: one label per sequence (reward models, rerankers, classifiers) and one label per
token (paddleformers/transformers/*/modeling.py ``...ForSequenceClassification`` / ``...ForTokenClassification``, e.g.
seed_oss, intern_lm2, gemma3_text, minicpm4_1).

``DecoderForSequenceClassification`` reads the hidden state of the last token that is not padding and applies a bias-free
``score`` projection; the loss follows ``problem_type``: mean squared error for one regression target, cross entropy for one label
out of several, binary cross entropy with logits for independent labels. ``DecoderForTokenClassification`` applies a biased
``score`` projection to every position. Both load the decoder weights of any causal-LM checkpoint of a supported family (the
language-model head is ignored, a missing ``score`` keeps its initial values).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..transformers.conversion_utils import Rule, WeightMap
from ..transformers.model_utils import PretrainedModel
from .configuration import DecoderConfig
from .modeling import DecoderModel, _resolve_dtype, build_weight_map


@dataclass
class ClassifierOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None


class _DecoderWithHead(PretrainedModel):
    config_class = DecoderConfig
    base_model_prefix = "model"
    head_bias = False

    def __init__(self, config: DecoderConfig, dtype=None, device=None):
        super().__init__(config)
        dtype = dtype if dtype is not None else _resolve_dtype(config.dtype)
        labels = getattr(config, "num_labels", None) or len(getattr(config, "id2label", None) or {}) or 2
        self.num_labels = config.num_labels = int(labels)          # checkpoints record the label set as ``id2label``
        self.model = DecoderModel(config, dtype=dtype, device=device)
        self.score = nn.Linear(config.hidden_size, self.num_labels, bias=self.head_bias, dtype=dtype, device=device)
        self.post_init()

    def _init_weights(self, module):
        std = self.config.initializer_range
        if isinstance(module, (nn.Linear, nn.Embedding)):
            nn.init.normal_(module.weight, 0.0, std)
            if getattr(module, "bias", None) is not None:
                nn.init.zeros_(module.bias)

    def hidden(self, input_ids, position_ids=None, kend=None):
        hidden, ctx = self.model(input_ids, position_ids, kend)
        if self.model.sp:
            # every rank holds a slice of the token rows: gather them (all ranks then compute the same head and loss, so the
            # backward pass keeps this rank's slice)
            from ..parallel.tensor_parallel import GatherOp
            from ..parallel.topology import get_parallel_state

            hidden = GatherOp.apply(hidden, get_parallel_state().group("mp"))
        return hidden.view(ctx.B, ctx.S, -1)

    def weight_map(self) -> WeightMap:
        own = dict(self.named_parameters())
        text_map = build_weight_map(self.config)
        rules = [r for r in text_map.rules.values() if r.target in own]
        known = {r.target for r in rules}
        rules += [Rule(n, [text_map.translate(n)]) for n in own if n not in known]
        return WeightMap(rules)


class DecoderForSequenceClassification(_DecoderWithHead):
    def forward(self, input_ids, labels=None, position_ids=None, attention_mask=None, **unused):
        h = self.hidden(input_ids, position_ids)
        B, S, _ = h.shape
        pad = getattr(self.config, "pad_token_id", None)
        if attention_mask is not None:
            keep = attention_mask.to(torch.bool)
        elif pad is not None:
            keep = input_ids != pad
        else:
            keep = torch.ones_like(input_ids, dtype=torch.bool)
        last = (torch.arange(S, device=input_ids.device)[None] * keep).argmax(dim=1)          # right-most kept position
        pooled = h[torch.arange(B, device=h.device), last]
        logits = self.score(pooled).float()
        out = ClassifierOutput(logits=logits, hidden_states=pooled)
        if labels is not None:
            kind = getattr(self.config, "problem_type", None)
            if kind is None:
                kind = "regression" if self.num_labels == 1 else \
                    ("single_label_classification" if labels.dtype in (torch.long, torch.int) else "multi_label_classification")
            if kind == "regression":
                out.loss = TF.mse_loss(logits.squeeze(-1) if self.num_labels == 1 else logits, labels.float().reshape(logits.squeeze(-1).shape
                                                                                                              if self.num_labels == 1 else logits.shape))
            elif kind == "single_label_classification":
                out.loss = TF.cross_entropy(logits, labels.reshape(-1))
            else:
                out.loss = TF.binary_cross_entropy_with_logits(logits, labels.float())
        return out


class DecoderForTokenClassification(_DecoderWithHead):
    head_bias = True

    def forward(self, input_ids, labels=None, position_ids=None, **unused):
        h = self.hidden(input_ids, position_ids)
        logits = self.score(h).float()
        out = ClassifierOutput(logits=logits)
        if labels is not None:
            out.loss = TF.cross_entropy(logits.view(-1, self.num_labels), labels.reshape(-1), ignore_index=-100)
        return out
