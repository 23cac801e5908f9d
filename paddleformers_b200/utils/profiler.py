"""Step-window profiling helpers.

* ``switch_profile(step, start, end)`` - brackets steps [start, end) with ``cudaProfilerStart`` / ``cudaProfilerStop`` so
  that an external profiler with capture-range = cudaProfilerApi records exactly that window
  (paddleformers/utils/perf_utils.py:83).
* ``TorchProfilerCallback`` - the same window recorded by ``torch.profiler`` and exported as a Chrome trace plus a table
  of the most expensive operators, for machines without an external profiler (paddleformers/utils/profiler.py).
* ``StartupTimer`` - wall-clock marks of the phases before the first step (imports, model build, data, first batch), logged
  once (paddleformers/trainer/startup_profile.py).
"""
from __future__ import annotations

import os
import time
from typing import Dict, Optional

import torch

from ..trainer.trainer_callback import TrainerCallback
from .log import logger

_profiling = False
_open_step_range = False


def switch_profile(step: int, start: int, end: int, enable_nvtx: bool = True) -> None:
    """Call once at the top of every step. Each step inside the window is one NVTX range ``step_<n>``; the range of the
    previous step is closed before the next one opens, and the last one before the profiler stops."""
    global _profiling, _open_step_range
    if not torch.cuda.is_available():
        return
    if _open_step_range:
        torch.cuda.nvtx.range_pop()
        _open_step_range = False
    if step == start and not _profiling:
        torch.cuda.cudart().cudaProfilerStart()
        _profiling = True
    if step == end and _profiling:
        torch.cuda.cudart().cudaProfilerStop()
        _profiling = False
    if _profiling and enable_nvtx and start <= step < end:
        torch.cuda.nvtx.range_push(f"step_{step}")
        _open_step_range = True


class NvtxModuleRanges:
    """Forward pre / post hooks that wrap every sub-module down to ``depth`` levels in an NVTX range named by its
    qualified name and class, plus full-backward hooks with a ``bwd:`` prefix, so that a timeline shows which layer a
    kernel belongs to (the reference registers such hooks when its profiler is on: paddleformers/utils/perf_utils.py).
    ``push`` / ``pop`` are injectable for tests; by default they are ``torch.cuda.nvtx.range_push`` / ``range_pop``."""

    def __init__(self, model: torch.nn.Module, depth: int = 3, backward: bool = True, push=None, pop=None):
        self.push = push or torch.cuda.nvtx.range_push
        self.pop = pop or torch.cuda.nvtx.range_pop
        self.handles = []
        for name, mod in model.named_modules():
            if name == "" or name.count(".") >= depth:
                continue
            label = f"{name}:{type(mod).__name__}"
            self.handles.append(mod.register_forward_pre_hook(lambda m, a, _l=label: self.push(_l)))
            self.handles.append(mod.register_forward_hook(lambda m, a, o, _l=label: self.pop(), always_call=True))
            if backward:
                self.handles.append(mod.register_full_backward_pre_hook(lambda m, g, _l=label: self.push("bwd:" + _l)))
                self.handles.append(mod.register_full_backward_hook(lambda m, gi, go, _l=label: self.pop()))

    def remove(self) -> None:
        for h in self.handles:
            h.remove()
        self.handles = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.remove()


class TorchProfilerCallback(TrainerCallback):
    def __init__(self, start_step: int = 3, end_step: int = 5, out_dir: Optional[str] = None, with_stack: bool = False):
        self.start, self.end, self.out_dir, self.with_stack = start_step, end_step, out_dir, with_stack
        self.prof = None
        self.trace_path: Optional[str] = None
        self.table: Optional[str] = None

    def on_step_begin(self, args, state, control, **kw):
        if state.global_step == self.start and self.prof is None:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self.prof = torch.profiler.profile(activities=acts, record_shapes=True, with_stack=self.with_stack)
            self.prof.__enter__()

    def on_step_end(self, args, state, control, **kw):
        if self.prof is not None and state.global_step >= self.end:
            self.prof.__exit__(None, None, None)
            out = self.out_dir or os.path.join(args.output_dir, "profile")
            os.makedirs(out, exist_ok=True)
            self.trace_path = os.path.join(out, f"trace_rank{args.process_index}.json")
            self.prof.export_chrome_trace(self.trace_path)
            key = "cuda_time_total" if torch.cuda.is_available() else "cpu_time_total"
            self.table = self.prof.key_averages().table(sort_by=key, row_limit=25)
            with open(os.path.join(out, f"top_ops_rank{args.process_index}.txt"), "w") as f:
                f.write(self.table)
            logger.info(f"profile of steps [{self.start}, {self.end}) written to {out}")
            self.prof = None
            self.start = 1 << 60          # once


class StartupTimer:
    def __init__(self):
        self.t0 = time.perf_counter()
        self.marks: Dict[str, float] = {}

    def mark(self, name: str):
        self.marks[name] = time.perf_counter() - self.t0

    def report(self) -> str:
        prev, parts = 0.0, []
        for k, v in self.marks.items():
            parts.append(f"{k}: {v - prev:.2f}s")
            prev = v
        msg = "startup: " + ", ".join(parts) + f" (total {prev:.2f}s)"
        logger.info(msg)
        return msg
