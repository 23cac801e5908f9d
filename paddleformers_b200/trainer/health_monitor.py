"""Training-health monitors: sampled statistics of activations, router load, gradients and weights, written as JSON lines.

The reference wires an optional external package ("internal medicine") into the trainer through
``InternalMedicineCallback`` (paddleformers/trainer/trainer_callback.py:966-1230): monitors are registered on the model, run
every ``monitor_interval`` steps, skip the first step after a resume, and rank 0 appends one record per sampled step to
``internal_medicine.jsonl`` (rotated aside on a fresh start, truncated to the resumed step on a resume). This module provides
the monitors themselves, so nothing external is needed:

* ``activations`` - RMS and absolute maximum of every decoder layer's output (forward hooks, sampled steps only);
* ``router``      - per MoE layer: largest expert share, share of idle experts, normalised entropy of the expert load since the
  last sample (from the router's usage counter);
* ``grads``       - global and per-layer gradient norms read from the fp32 accumulation buffers at the optimizer boundary;
* ``weights``     - per-layer weight norms and the norm of the stacked expert weights.

Every statistic stays on the device until the record is written; only sampled steps synchronise.
"""
from __future__ import annotations

import json
import os
import re
import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.log import logger
from .trainer_callback import TrainerCallback

ALL_MONITORS = ("activations", "router", "grads", "weights")
_LAYER = re.compile(r"layers\.(\d+)\.")


class HealthMonitorCallback(TrainerCallback):
    def __init__(self, monitors=None, monitor_interval: int = 0, log_dir: str = "", file_name: str = "internal_medicine.jsonl"):
        if monitors is None or monitors == "all" or monitors == ["all"]:
            monitors = list(ALL_MONITORS)
        if isinstance(monitors, str):
            monitors = [m.strip() for m in monitors.split(",") if m.strip()]
        unknown = [m for m in monitors if m not in ALL_MONITORS]
        if unknown:
            raise ValueError(f"unknown monitors {unknown}; choose from {ALL_MONITORS}")
        self.monitors = list(monitors)
        self.interval = int(monitor_interval or 0)
        self.log_path = os.path.join(log_dir, file_name) if log_dir else ""
        self._handles: List = []
        self._sampling = False
        self._skip = 0
        self._record: Dict[str, torch.Tensor] = {}
        self._usage_prev: Dict[str, torch.Tensor] = {}
        self.records: List[Dict[str, float]] = []

    # ------------------------------------------------------------------ life cycle
    def _is_writer(self) -> bool:
        return bool(self.log_path) and (not dist.is_initialized() or dist.get_rank() == 0)

    def on_train_begin(self, args, state, control, model=None, **kw):
        if self.interval <= 0 or model is None:
            return
        self._prepare_file(int(state.global_step or 0))
        if state.global_step:
            self._skip = 1            # the first step after a resume re-builds caches and graphs: do not sample it
        if "activations" in self.monitors and not self._handles:
            for name, mod in model.named_modules():
                if re.fullmatch(r"(.*\.)?layers\.\d+", name):
                    self._handles.append(mod.register_forward_hook(self._make_hook(int(name.rsplit(".", 1)[1]))))

    def on_train_end(self, args, state, control, **kw):
        for h in self._handles:
            h.remove()
        self._handles = []

    def _prepare_file(self, resume_step: int) -> None:
        if not self._is_writer() or not os.path.exists(self.log_path):
            return
        if resume_step <= 0:          # fresh start: move the previous run's file out of the way
            bak = f"{self.log_path}.bak.{time.strftime('%Y%m%d_%H%M%S')}"
            n = 0
            while os.path.exists(bak + (f".{n}" if n else "")):
                n += 1
            os.replace(self.log_path, bak + (f".{n}" if n else ""))
            return
        kept = []
        with open(self.log_path, encoding="utf-8") as f:
            for line in f:
                line = line.rstrip("\n")
                if not line:
                    continue
                try:
                    if int(json.loads(line).get("global_step", 0)) <= resume_step:
                        kept.append(line)
                except (json.JSONDecodeError, ValueError, TypeError):
                    kept.append(line)                 # keep what cannot be parsed rather than drop it silently
        with open(self.log_path, "w", encoding="utf-8") as f:
            f.write("".join(l + "\n" for l in kept))

    # ------------------------------------------------------------------ sampling
    def on_step_begin(self, args, state, control, **kw):
        if self.interval <= 0:
            return
        if self._skip > 0:
            self._skip -= 1
            self._sampling = False
            return
        self._sampling = (state.global_step + 1) % self.interval == 0
        self._record = {}

    def _make_hook(self, layer: int):
        def hook(mod, args, out):
            if not self._sampling:
                return
            t = out[0] if isinstance(out, (tuple, list)) else out
            if isinstance(out, (tuple, list)) and len(out) > 1 and torch.is_tensor(out[1]):
                t = t + out[1]                        # (branch output, residual stream): the layer's output is their sum
            t = t.detach().float()
            # several micro-batches per step: keep the largest value seen
            for key, val in ((f"act_rms/layer{layer}", t.pow(2).mean().sqrt()), (f"act_absmax/layer{layer}", t.abs().max())):
                self._record[key] = torch.maximum(self._record[key], val) if key in self._record else val
        return hook

    def on_optimizer_begin(self, args, state, control, model=None, **kw):
        if not self._sampling or model is None:
            return
        rec = self._record
        if "grads" in self.monitors or "weights" in self.monitors:
            g_layers: Dict[str, List[torch.Tensor]] = {}
            w_layers: Dict[str, List[torch.Tensor]] = {}
            for name, p in model.named_parameters():
                m = _LAYER.search(name)
                key = f"layer{m.group(1)}" if m else "other"
                g = getattr(p, "main_grad", None)
                if g is None:
                    g = p.grad
                if g is not None and "grads" in self.monitors:
                    g_layers.setdefault(key, []).append(g.detach().float().pow(2).sum())
                if "weights" in self.monitors:
                    w_layers.setdefault(key, []).append(p.detach().float().pow(2).sum())
                    if getattr(p, "is_expert", False):
                        rec[f"expert_weight_norm/{key}/{name.rsplit('.', 1)[-1]}"] = p.detach().float().norm()
            for key, parts in g_layers.items():
                rec[f"grad_norm/{key}"] = torch.stack(parts).sum().sqrt()
            if g_layers:
                rec["grad_norm/all"] = torch.stack([torch.stack(v).sum() for v in g_layers.values()]).sum().sqrt()
            for key, parts in w_layers.items():
                rec[f"weight_norm/{key}"] = torch.stack(parts).sum().sqrt()
        if "router" in self.monitors:
            for name, mod in model.named_modules():
                usage = getattr(mod, "expert_usage", None)
                if usage is None or not torch.is_tensor(usage):
                    continue
                m = _LAYER.search(name + ".")
                key = f"layer{m.group(1)}" if m else name
                prev = self._usage_prev.get(name)
                cur = usage.detach().clone()
                delta = (cur - prev) if prev is not None and bool((cur >= prev).all()) else cur   # the counter may be reset
                self._usage_prev[name] = cur
                load = delta.float() / delta.float().sum().clamp_min(1.0)
                E = load.numel()
                rec[f"router_max_share/{key}"] = load.max() * E              # 1.0 = perfectly even
                rec[f"router_idle_share/{key}"] = (delta == 0).float().mean()
                ent = -(load * torch.log(load.clamp_min(1e-20))).sum() / torch.log(torch.tensor(float(E)))
                rec[f"router_entropy/{key}"] = ent

    def on_step_end(self, args, state, control, **kw):
        if not self._sampling:
            return
        self._sampling = False
        out = {"global_step": int(state.global_step)}
        out.update({k: round(float(v), 6) for k, v in sorted(self._record.items())})
        self._record = {}
        self.records.append(out)
        if self._is_writer():
            os.makedirs(os.path.dirname(self.log_path) or ".", exist_ok=True)
            with open(self.log_path, "a", encoding="utf-8") as f:
                f.write(json.dumps(out) + "\n")
        bad = [k for k, v in out.items() if isinstance(v, float) and v != v]
        if bad:
            logger.warning(f"health monitor: NaN in {bad[:4]} at step {state.global_step}")
