"""Exponential moving average of the weights, kept on the optimizer shards.

Each rank averages only the fp32 master slice it owns (the same partition as the Adam moments), so the EMA costs
4 bytes / parameter / sharding-degree and one fused ``lerp`` per domain and step. ``export_ema_weights`` assembles a full
Hugging Face checkpoint from the shards by swapping them into the master buffers, re-gathering the working weights,
saving, and swapping back - the job of the reference's ``EMAStateAssembler``
(paddleformers/trainer/trainer_utils.py:1941) and EMA callback (paddleformers/trainer/trainer_callback.py).
"""
from __future__ import annotations

import os
from typing import Dict, List

import torch

from .trainer_callback import TrainerCallback


class EMACallback(TrainerCallback):
    def __init__(self, decay: float = 0.999, start_step: int = 0, interval: int = 1, loss_threshold: float = None):
        """``interval``: average every that many optimizer steps; ``loss_threshold``: average only while the last logged
        training loss is below it (``zcc_ema_interval`` / ``zcc_ema_loss_threshold`` of the reference's zero-cost
        checkpoint EMA, paddleformers/trainer/training_args.py:1225-1238; the reference keeps the average in its
        checkpoint worker's host memory, here it lives beside the master shard it averages)."""
        assert 0.0 < decay < 1.0
        self.decay, self.start_step = decay, start_step
        self.interval, self.loss_threshold = max(int(interval or 1), 1), loss_threshold
        self.shadow: Dict[str, torch.Tensor] = {}
        self.num_updates = 0
        self.last_loss = None

    def on_log(self, args, state, control, logs=None, **kw):
        if logs and "loss" in logs:
            self.last_loss = float(logs["loss"])

    def _domains(self, optimizer) -> List:
        return list(getattr(optimizer, "domains", []))

    def on_optimizer_end(self, args, state, control, optimizer=None, **kw):
        if optimizer is None or state.global_step + 1 < self.start_step or (state.global_step + 1) % self.interval != 0:
            return
        if self.loss_threshold is not None and self.last_loss is not None and not self.last_loss < self.loss_threshold:
            return
        with torch.no_grad():
            for dom in self._domains(optimizer):
                if dom.name not in self.shadow:
                    self.shadow[dom.name] = dom.master.detach().clone()
                else:
                    self.shadow[dom.name].lerp_(dom.master, 1.0 - self.decay)
        self.num_updates += 1

    # ---- checkpointing
    def state_dict(self) -> Dict[str, object]:
        return {"decay": self.decay, "num_updates": self.num_updates, "shadow": {k: v.cpu() for k, v in self.shadow.items()}}

    def load_state_dict(self, sd: Dict[str, object]):
        self.decay, self.num_updates = float(sd["decay"]), int(sd["num_updates"])
        for k, v in sd["shadow"].items():
            self.shadow[k] = v.to(self.shadow[k].device) if k in self.shadow else v

    def on_save(self, args, state, control, **kw):
        from .trainer_utils import PREFIX_CHECKPOINT_DIR

        out = os.path.join(args.output_dir, f"{PREFIX_CHECKPOINT_DIR}-{state.global_step}")
        if self.shadow and os.path.isdir(out):
            torch.save(self.state_dict(), os.path.join(out, f"ema_state_{args.process_index}.pt"))


def export_ema_weights(trainer, ema: EMACallback, out_dir: str) -> str:
    """Write the averaged weights as a Hugging Face directory (collective over the model-parallel and sharding groups)."""
    opt = trainer.optimizer
    saved = {}
    with torch.no_grad():
        for dom in opt.domains:
            if dom.name in ema.shadow:
                saved[dom.name] = dom.master.clone()
                dom.master.copy_(ema.shadow[dom.name].to(dom.master.device))
        opt.load_state_dict(_as_state(opt))          # rebuilds (and all-gathers) the working weights from the masters
        trainer.model.save_pretrained(out_dir)
        for dom in opt.domains:
            if dom.name in saved:
                dom.master.copy_(saved[dom.name])
        opt.load_state_dict(_as_state(opt))
    return out_dir


def _as_state(opt) -> Dict[str, object]:
    return {"step": opt.step_count, "lr": opt.lr,
            "domains": {d.name: {"master": d.master, "exp_avg": d.exp_avg, "exp_avg_sq": d.exp_avg_sq, "shard_size": d.shard_size,
                                 "numel": d.numel} for d in opt.domains}}
