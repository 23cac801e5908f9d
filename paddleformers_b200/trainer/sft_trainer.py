"""Supervised fine-tuning trainer: the base loop plus perplexity in the training log and generation-based
evaluation, as in paddleformers/cli/train/sft/sft_trainer.py:58."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .trainer import Trainer


class SFTTrainer(Trainer):
    def __init__(self, *args, do_generation: bool = False, generation_kwargs: Optional[dict] = None, **kw):
        super().__init__(*args, **kw)
        self.do_generation = do_generation
        self.generation_kwargs = generation_kwargs or {"max_new_tokens": 64}

    def log(self, logs: Dict[str, float]):
        if "loss" in logs:
            logs = dict(logs, ppl=round(math.exp(min(float(logs["loss"]), 50.0)), 4))
        super().log(logs)

    @torch.no_grad()
    def generate_predictions(self, prompts: List[List[int]]) -> List[List[int]]:
        from ..generation.utils import generate

        self.model.eval()
        outs = []
        for p in prompts:
            ids = torch.tensor([p], device=self.device)
            outs.append(generate(self.model, ids, **self.generation_kwargs)[0, len(p):].tolist())
        self.model.train()
        return outs
