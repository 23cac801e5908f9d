"""Callback event bus of the trainer and the built-in callbacks.

Event names and control-flow object follow the reference (paddleformers/trainer/trainer_callback.py:232-370
TrainerCallback, :372 CallbackHandler, :508 DefaultFlowCallback); built-ins cover progress / logging, early stopping,
the aux-loss-free MoE bias update (:788-840), the fp8 weight re-quantisation hook (:722-785) and step-window
profiling (paddleformers/utils/perf_utils.py:83).
"""
from __future__ import annotations

import dataclasses
import json
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.log import logger


@dataclass
class TrainerState:
    epoch: float = 0.0
    global_step: int = 0
    max_steps: int = 0
    num_train_epochs: int = 0
    consumed_samples: int = 0
    total_flos: float = 0.0
    trained_tokens: int = 0
    log_history: List[Dict[str, float]] = field(default_factory=list)
    best_metric: Optional[float] = None
    best_model_checkpoint: Optional[str] = None
    is_world_process_zero: bool = True

    def save_to_json(self, path: str):
        with open(path, "w") as f:
            json.dump(dataclasses.asdict(self), f, indent=2, sort_keys=True)

    @classmethod
    def load_from_json(cls, path: str):
        with open(path) as f:
            return cls(**json.load(f))


@dataclass
class TrainerControl:
    should_training_stop: bool = False
    should_epoch_stop: bool = False
    should_save: bool = False
    should_evaluate: bool = False
    should_log: bool = False

    def _new_step(self):
        self.should_save = self.should_evaluate = self.should_log = False


class TrainerCallback:
    def on_init_end(self, args, state, control, **kw): pass
    def on_train_begin(self, args, state, control, **kw): pass
    def on_train_end(self, args, state, control, **kw): pass
    def on_epoch_begin(self, args, state, control, **kw): pass
    def on_epoch_end(self, args, state, control, **kw): pass
    def on_load_data_end(self, args, state, control, **kw): pass
    def on_step_begin(self, args, state, control, **kw): pass
    def on_substep_end(self, args, state, control, **kw): pass
    def on_optimizer_begin(self, args, state, control, **kw): pass
    def on_optimizer_end(self, args, state, control, **kw): pass
    def on_step_end(self, args, state, control, **kw): pass
    def on_evaluate(self, args, state, control, **kw): pass
    def on_save(self, args, state, control, **kw): pass
    def on_log(self, args, state, control, logs=None, **kw): pass
    def on_prediction_step(self, args, state, control, **kw): pass


class CallbackHandler(TrainerCallback):
    def __init__(self, callbacks, model, optimizer, lr_scheduler):
        self.callbacks: List[TrainerCallback] = []
        for cb in callbacks:
            self.add_callback(cb)
        self.model, self.optimizer, self.lr_scheduler = model, optimizer, lr_scheduler
        self.train_dataloader = None

    def add_callback(self, cb):
        cb = cb() if isinstance(cb, type) else cb
        if any(type(c) is type(cb) for c in self.callbacks):
            logger.warning(f"callback {type(cb).__name__} registered twice")
        self.callbacks.append(cb)

    def remove_callback(self, cb):
        self.callbacks = [c for c in self.callbacks if not (c is cb or (isinstance(cb, type) and isinstance(c, cb)))]

    def call_event(self, event, args, state, control, **kw):
        for cb in self.callbacks:
            res = getattr(cb, event)(args, state, control, model=self.model, optimizer=self.optimizer,
                                     lr_scheduler=self.lr_scheduler, train_dataloader=self.train_dataloader, **kw)
            if res is not None:
                control = res
        return control

    def __getattribute__(self, name):
        if name.startswith("on_"):
            return lambda args, state, control, **kw: object.__getattribute__(self, "call_event")(name, args, state, control, **kw)
        return object.__getattribute__(self, name)


class DefaultFlowCallback(TrainerCallback):
    """Decides when to log / evaluate / save / stop from the interval strategies."""

    def on_step_end(self, args, state, control, **kw):
        if state.global_step == 1 and args.logging_first_step:
            control.should_log = True
        if args.logging_steps > 0 and state.global_step % args.logging_steps == 0:
            control.should_log = True
        if args.eval_strategy == "steps" and args.eval_steps and state.global_step % args.eval_steps == 0:
            control.should_evaluate = True
        if args.save_strategy == "steps" and args.save_steps > 0 and state.global_step % args.save_steps == 0:
            control.should_save = True
        if state.global_step >= state.max_steps:
            control.should_training_stop = True
        return control

    def on_epoch_end(self, args, state, control, **kw):
        if args.eval_strategy == "epoch":
            control.should_evaluate = True
        if args.save_strategy == "epoch":
            control.should_save = True
        return control


class PrinterCallback(TrainerCallback):
    def on_log(self, args, state, control, logs=None, **kw):
        if state.is_world_process_zero and logs is not None:
            logger.train(", ".join(f"{k}: {v:.6g}" if isinstance(v, float) else f"{k}: {v}" for k, v in logs.items()))


class MetricsDumpCallback(TrainerCallback):
    """Appends every log record to a JSON-lines file (``metrics_output_path``)."""

    def __init__(self, path: str):
        from ..utils.log import MetricsDumper

        self.dumper = MetricsDumper(path)

    def on_log(self, args, state, control, logs=None, **kw):
        if logs is not None:
            self.dumper.append(dict(logs, global_step=state.global_step))

    def on_train_end(self, args, state, control, **kw):
        self.dumper.close()


class EarlyStoppingCallback(TrainerCallback):
    def __init__(self, patience: int = 3, threshold: float = 0.0, metric: str = "eval_loss", greater_is_better=False):
        self.patience, self.threshold, self.metric, self.gib = patience, threshold, metric, greater_is_better
        self.best, self.bad = None, 0

    def on_evaluate(self, args, state, control, metrics=None, **kw):
        if not metrics or self.metric not in metrics:
            return
        v = metrics[self.metric]
        better = self.best is None or ((v > self.best + self.threshold) if self.gib else (v < self.best - self.threshold))
        if better:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                control.should_training_stop = True
        return control


class MoECorrectionBiasAdjustCallback(TrainerCallback):
    """Aux-loss-free load balancing: after each optimizer step, experts that received more than the mean number of
    tokens get their selection bias lowered by ``update_rate`` and the others raised; the usage counters are summed
    over every rank that routed different tokens first (paddleformers/trainer/trainer_callback.py:788-840)."""

    def __init__(self, update_rate: float = 1e-3):
        self.update_rate = update_rate

    def on_optimizer_end(self, args, state, control, model=None, **kw):
        from ..nn.moe import TopkRouter

        routers = [m for m in model.modules() if isinstance(m, TopkRouter) and m.e_score_correction_bias is not None]
        if not routers:
            return
        usage = torch.stack([r.expert_usage for r in routers]).to(torch.float32)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(usage)
        mean = usage.mean(-1, keepdim=True)
        delta = torch.sign(mean - usage) * self.update_rate
        for r, d in zip(routers, delta):
            r.e_score_correction_bias.add_(d.to(r.e_score_correction_bias.dtype))
            r.expert_usage.zero_()


class FP8QuantWeightCallback(TrainerCallback):
    """Refreshes cached fp8 copies of the weights after every optimizer step so that the next forward reads
    quantised weights consistent with the updated bf16 / fp32 masters
    (paddleformers/trainer/trainer_callback.py:722-785)."""

    def on_optimizer_end(self, args, state, control, model=None, **kw):
        for m in model.modules():
            refresh = getattr(m, "refresh_fp8_weight_cache", None)
            if refresh is not None:
                refresh()

    on_train_begin = on_optimizer_end


class ProfilerCallback(TrainerCallback):
    """Brackets steps [profile_step_start, profile_step_end) with cudaProfilerStart/Stop and one NVTX range per
    step, so that ``ncu`` / ``nsys`` with capture-range = cudaProfilerApi record exactly those steps."""

    def on_step_begin(self, args, state, control, **kw):
        if not (args.profile and torch.cuda.is_available()):
            return
        step = state.global_step
        if step == args.profile_step_start:
            torch.cuda.cudart().cudaProfilerStart()
            depth = int(getattr(args, "profile_nvtx_depth", 0) or 0)
            if depth > 0 and kw.get("model") is not None:
                from ..utils.profiler import NvtxModuleRanges

                self._ranges = NvtxModuleRanges(kw["model"], depth=depth)   # one range per sub-module, forward and backward
        if args.profile_step_start <= step < args.profile_step_end:
            torch.cuda.nvtx.range_push(f"step_{step}")

    def on_step_end(self, args, state, control, **kw):
        if not (args.profile and torch.cuda.is_available()):
            return
        step = state.global_step - 1
        if args.profile_step_start <= step < args.profile_step_end:
            torch.cuda.nvtx.range_pop()
        if step + 1 == args.profile_step_end:
            torch.cuda.cudart().cudaProfilerStop()
            if getattr(self, "_ranges", None) is not None:
                self._ranges.remove()
                self._ranges = None
