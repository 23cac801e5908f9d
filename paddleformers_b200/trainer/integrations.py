"""Reporting callbacks selected by ``TrainingArguments.report_to``.

* ``tensorboard`` — scalars through ``torch.utils.tensorboard`` when the ``tensorboard`` package is importable,
  otherwise through ``JsonlScalarWriter`` (same call surface), so a run never fails for a missing logger.
* ``visualdl`` / ``jsonl`` — scalars as JSON lines (``<logging_dir>/scalars.jsonl``): the role VisualDL's LogWriter plays
  for the reference (paddleformers/trainer/integrations.py:83 VisualDLCallback).
* ``TimerCallback`` — brackets data loading, forward + backward and the optimizer step with ``utils.timer.Timers`` and
  adds their per-step means to every log record (paddleformers/trainer/plugins/timer.py:100).
* ``MemoryCallback`` — device memory high-water marks in every log record
  (paddleformers/trainer/trainer_utils.py:961 TrainerMemoryTracker).

Only the global first rank writes; every rank keeps timers so that slow ranks can be found from their own logs.
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional

import torch

from ..utils.timer import Timers, set_timers
from .trainer_callback import TrainerCallback


class JsonlScalarWriter:
    """``add_scalar(tag, value, step)`` appended as one JSON object per line."""

    def __init__(self, logdir: str):
        os.makedirs(logdir, exist_ok=True)
        self.path = os.path.join(logdir, "scalars.jsonl")
        self._f = open(self.path, "a", buffering=1)

    def add_scalar(self, tag: str, value, step: int):
        self._f.write(json.dumps({"tag": tag, "value": float(value), "step": int(step), "time": time.time()}) + "\n")

    def add_text(self, tag: str, text: str, step: int = 0):
        self._f.write(json.dumps({"tag": tag, "text": text, "step": int(step), "time": time.time()}) + "\n")

    def flush(self):
        self._f.flush()

    def close(self):
        self._f.close()


def _make_writer(kind: str, logdir: str):
    if kind == "tensorboard":
        try:
            from torch.utils.tensorboard import SummaryWriter

            return SummaryWriter(log_dir=logdir)
        except Exception:  # noqa: BLE001 - package missing: keep the scalars anyway
            return JsonlScalarWriter(logdir)
    return JsonlScalarWriter(logdir)


class ScalarReportCallback(TrainerCallback):
    def __init__(self, kind: str = "jsonl", logdir: Optional[str] = None):
        self.kind, self.logdir, self.writer = kind, logdir, None

    def on_train_begin(self, args, state, control, **kw):
        if not state.is_world_process_zero:
            return
        logdir = self.logdir or getattr(args, "logging_dir", None) or os.path.join(args.output_dir, "runs")
        self.writer = _make_writer(self.kind, logdir)
        self.writer.add_text("args", json.dumps({k: v for k, v in vars(args).items() if isinstance(v, (int, float, str, bool))}))

    def on_log(self, args, state, control, logs=None, **kw):
        if self.writer is None or not logs:
            return
        for k, v in logs.items():
            if isinstance(v, (int, float)):
                self.writer.add_scalar(f"train/{k}" if not k.startswith("eval_") else f"eval/{k[5:]}", v, state.global_step)
        self.writer.flush()

    def on_train_end(self, args, state, control, **kw):
        if self.writer is not None:
            self.writer.close()
            self.writer = None


class TensorBoardCallback(ScalarReportCallback):
    def __init__(self, logdir: Optional[str] = None):
        super().__init__("tensorboard", logdir)


class VisualDLCallback(ScalarReportCallback):
    def __init__(self, logdir: Optional[str] = None):
        super().__init__("jsonl", logdir)


class TimerCallback(TrainerCallback):
    """data-load / forward-backward / optimizer-step timers; their per-step means go into the log record."""

    def __init__(self):
        self.timers: Optional[Timers] = None
        self._steps = 0

    def on_train_begin(self, args, state, control, **kw):
        self.timers = set_timers(Timers(use_cuda=str(args.device).startswith("cuda") and torch.cuda.is_available()))
        self.timers("read-data").start()

    def on_load_data_end(self, args, state, control, **kw):
        t = self.timers("read-data")
        if t._open is not None:
            t.stop()
        fb = self.timers("forward-backward")
        if fb._open is None:
            fb.start()

    def on_substep_end(self, args, state, control, **kw):
        self.timers("read-data").start()

    def on_optimizer_begin(self, args, state, control, **kw):
        self.timers("forward-backward").stop()
        self.timers("optimizer-step").start()

    def on_optimizer_end(self, args, state, control, **kw):
        self.timers("optimizer-step").stop()
        self._steps += 1
        self.timers("read-data").start()

    def augment_logs(self, args, state, logs):
        if logs is None or self.timers is None or "loss" not in logs:
            return
        rd = self.timers("read-data")
        running = rd._open is not None
        if running:
            rd.stop()
        for k, v in self.timers.info(normalizer=max(self._steps, 1)).items():
            logs[f"timer_{k.replace('-', '_')}_ms"] = round(v, 3)
        self._steps = 0
        if running:
            rd.start()


class MemoryCallback(TrainerCallback):
    def augment_logs(self, args, state, logs):
        if logs is None or not torch.cuda.is_available() or "loss" not in logs:
            return
        gib = float(1 << 30)
        logs["max_memory_allocated_gb"] = round(torch.cuda.max_memory_allocated() / gib, 3)
        logs["max_memory_reserved_gb"] = round(torch.cuda.max_memory_reserved() / gib, 3)


def callbacks_from_args(args) -> List[TrainerCallback]:
    """Callbacks for ``report_to`` ("none" | comma-separated subset of tensorboard, visualdl, jsonl) plus the timer and
    memory callbacks when ``enable_timer`` / ``log_memory`` are set."""
    out: List[TrainerCallback] = []
    names = [n.strip() for n in str(getattr(args, "report_to", "none") or "none").split(",")]
    for n in names:
        if n in ("none", ""):
            continue
        if n == "tensorboard":
            out.append(TensorBoardCallback())
        elif n in ("visualdl", "jsonl"):
            out.append(VisualDLCallback())
        else:
            raise ValueError(f"report_to: unknown logger {n!r} (tensorboard, visualdl, jsonl, none)")
    zcc_coef = getattr(args, "zcc_save_ema_coef", None) if getattr(args, "enable_zero_cost_checkpoint", False) else None
    if float(getattr(args, "ema_decay", 0.0) or 0.0) > 0 or (zcc_coef is not None and 0.0 < float(zcc_coef) < 1.0):
        from .ema import EMACallback

        decay = float(args.ema_decay) if float(getattr(args, "ema_decay", 0.0) or 0.0) > 0 else float(zcc_coef)
        out.append(EMACallback(decay, int(getattr(args, "ema_start_step", 0) or 0),
                               interval=int(getattr(args, "zcc_ema_interval", 1) or 1),
                               loss_threshold=getattr(args, "zcc_ema_loss_threshold", None)))
    if int(getattr(args, "internal_medicine_monitor_interval", 0) or 0) > 0:
        from .health_monitor import HealthMonitorCallback

        out.append(HealthMonitorCallback(getattr(args, "internal_medicine_monitors", None) or "all",
                                         int(args.internal_medicine_monitor_interval),
                                         log_dir=getattr(args, "logging_dir", None) or os.path.join(args.output_dir, "runs")))
    if getattr(args, "flash_device_path", None):
        from ..utils.ckpt_mirror import MirrorCallback

        out.append(MirrorCallback(args.flash_device_path))
    if getattr(args, "enable_timer", False):
        out.append(TimerCallback())
    if getattr(args, "log_memory", False):
        out.append(MemoryCallback())
    return out
